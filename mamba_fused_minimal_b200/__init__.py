"""B200-native Mamba2 SSD forward hot path behind the call surface of
RishiAstra/mamba-fused-minimal.

    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd, _chunk_state_fwd
    from mamba_fused_minimal_b200.kernels.ssd_state_passing import _state_passing_fwd
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent
    from mamba_fused_minimal_b200.kernels.fused_globalbar import _fused_chunk_state_state_passing_fwd_globalbar
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _chunk_scan_fwd

The module names and function names are the reference's (its `kernels/` package and
`main.py`); every function runs hand-written sm_100a CUDA through the C ABI in
include/ssd_b200.h.  Importing the kernels needs the prebuilt native modules
(`python -m mamba_fused_minimal_b200.build`); there is no fallback path.
"""
__version__ = "0.1.0"
