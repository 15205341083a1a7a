"""`_fused_chunk_state_state_passing_fwd_concurrent` with the reference's signature
(kernels/fused_concurrent.py:255-331): per-chunk state and state passing in one launch,
returning (out (batch, nchunks, nheads, headdim, dstate) in out_dtype,
final_states (batch, nheads, headdim, dstate) fp32).

Differences a caller can observe: no text is printed, the device is the inputs' device
rather than "cuda", the waits inside the kernel are bounded, and the fp32 per-chunk states
are only written when a `states` buffer is passed."""
from ._fused import _fused_chunk_state_state_passing_fwd


def _fused_chunk_state_state_passing_fwd_concurrent(B, x, dt, dA_cumsum, out_dtype, initial_states=None,
                                                    seq_idx=None, states=None, states_in_fp32=True):
    return _fused_chunk_state_state_passing_fwd(B, x, dt, dA_cumsum, out_dtype, initial_states, seq_idx,
                                                states, states_in_fp32)
