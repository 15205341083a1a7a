"""`_fused_chunk_state_state_passing_fwd_globalbar` with the reference's signature
(kernels/fused_globalbar.py:201-266).  The reference has two fused kernels that differ in
how they synchronise (a grid-wide barrier there, overlapped phases in fused_concurrent);
both names map to the same kernel here, which needs neither."""
from ._fused import _fused_chunk_state_state_passing_fwd


def _fused_chunk_state_state_passing_fwd_globalbar(B, x, dt, dA_cumsum, out_dtype, initial_states=None,
                                                   seq_idx=None, states=None, states_in_fp32=True):
    return _fused_chunk_state_state_passing_fwd(B, x, dt, dA_cumsum, out_dtype, initial_states, seq_idx,
                                                states, states_in_fp32)
