"""The whole state path in one call: chunk cumsum, per-chunk state and inter-chunk state passing.

The reference's pipelines make two calls for it (main.py:96-100 there): `_chunk_cumsum_fwd`
(kernels/ssd_chunk_state.py:176-199) and then one of the fused entry points
(kernels/fused_concurrent.py:255-331, kernels/fused_globalbar.py:201-266).  `_state_path_fwd` gives
the four tensors those two calls give, bit for bit, from ONE kernel launch where the tcgen05 state
kernel takes the problem: the persistent kernel computes each chunk's cumulative sums in the warp
that needs them and writes dt_out / dA_cumsum as a by-product.  Argument names follow the two
reference functions."""
from .._ext import C as _C


def _state_path_fwd(dt, A, B, x, chunk_size, out_dtype, dt_bias=None, dt_softplus=False,
                    dt_limit=(0.0, float("inf")), initial_states=None, seq_idx=None, states=None,
                    states_in_fp32=True, final_states=None):
    """dt (batch, seqlen, nheads) raw, A (nheads,), B (batch, seqlen, ngroups, dstate),
    x (batch, seqlen, nheads, headdim) -> (dA_cumsum, dt_out, out, final_states): the pair
    `_chunk_cumsum_fwd` returns followed by the pair the fused entry points return."""
    batch, seqlen, nheads, headdim = x.shape
    _, _, ngroups, dstate = B.shape
    assert dt.shape == (batch, seqlen, nheads)
    assert A.shape == (nheads,)
    if dt_bias is not None:
        assert dt_bias.shape == (nheads,)
    assert nheads % ngroups == 0
    assert B.shape == (batch, seqlen, ngroups, dstate)
    nchunks = (seqlen + chunk_size - 1) // chunk_size
    if seq_idx is not None:
        assert seq_idx.shape == (batch, seqlen)
    if states is not None:
        assert states.shape == (batch, nchunks, nheads, headdim, dstate)
    if initial_states is not None:
        assert initial_states.shape == (batch, nheads, headdim, dstate)
    return _C.state_path_fwd(dt, A, B, x, int(chunk_size), out_dtype, dt_bias, bool(dt_softplus),
                             float(dt_limit[0]), float(dt_limit[1]), initial_states, seq_idx, states,
                             bool(states_in_fp32), True, False, final_states)
