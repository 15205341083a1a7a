"""Multi-GPU partitioning of the SSD state path.  One process per GPU (torch.distributed).

Heads and batch shard with no communication: every kernel is independent per (batch, head)
given its group's B, so a rank simply calls the single-GPU functions on its shard
(`shard_heads`, `shard_batch` say which).

A long sequence shards along the sequence.  The recurrence over chunks is affine in the
carried state, S -> P * S + Z, so each rank scans its slice with a zero carry-in, the ranks
exchange their slice summaries (Z: the slice-final state, log P: the slice's summed
log-decay; 2.6 MB per rank at 80 heads), and a fix-up pass adds the carried state to the local
passed states (`seqpar_fused_state_fwd`).  The exchange is one all-gather over NCCL; the
gathered buffer is local memory, from which the fix-up kernel forms its own carry-in.

The reference is single-GPU (device hard-coded, kernels/fused_concurrent.py:289); what makes
sharding possible there is the initial_states / final_states pair
(kernels/ssd_state_passing.py:61-65,81), which this module composes across ranks.
"""
import torch
import torch.distributed as dist


def shard_range(n, world, rank):
    """Contiguous, near-equal split of range(n): (start, stop) of `rank`."""
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def shard_heads(nheads, ngroups, world, rank):
    """Head range of `rank` and the matching group range.  Heads of one B/C group stay on one
    GPU whenever there are at least `world` groups; with fewer groups (e.g. one) the heads are
    split and every rank keeps the whole group tensor."""
    ratio = nheads // ngroups
    if ngroups >= world:
        g0, g1 = shard_range(ngroups, world, rank)
        return (g0 * ratio, g1 * ratio), (g0, g1)
    h0, h1 = shard_range(nheads, world, rank)
    return (h0, h1), (h0 // ratio, (h1 - 1) // ratio + 1)


def shard_batch(batch, world, rank):
    return shard_range(batch, world, rank)


def shard_sequence(seqlen, chunk_size, world, rank):
    """Chunk-aligned slice [start, stop) of the sequence for `rank` (whole chunks per rank, the
    ragged last chunk on the last rank that has any)."""
    nchunks = (seqlen + chunk_size - 1) // chunk_size
    c0, c1 = shard_range(nchunks, world, rank)
    return min(c0 * chunk_size, seqlen), min(c1 * chunk_size, seqlen)


def summary_buffer(batch, nheads, headdim, dstate, device):
    """One rank's slice summary as a single fp32 buffer, so that one collective moves it:
    returns (buf, Z, logP) where Z (b, h, p, n) and logP (b, h) are views into buf."""
    nz = batch * nheads * headdim * dstate
    buf = torch.empty(nz + batch * nheads, dtype=torch.float32, device=device)
    return buf, buf[:nz].view(batch, nheads, headdim, dstate), buf[nz:].view(batch, nheads)


def exchange_summaries(buf, shape, group=None):
    """All-gather the ranks' summary buffers (from `summary_buffer`, shape = (b, h, p, n)).
    Returns (Z_all (world, b, h, p, n), logP_all (world, b, h)): views into the one gathered,
    local buffer."""
    world = dist.get_world_size(group)
    b, h, p, n = shape
    nz = b * h * p * n
    gathered = torch.empty(world * buf.numel(), dtype=buf.dtype, device=buf.device)
    dist.all_gather_into_tensor(gathered, buf, group=group)
    g = gathered.view(world, buf.numel())
    Z_all = g[:, :nz].unflatten(1, (b, h, p, n))
    logP_all = g[:, nz:].unflatten(1, (b, h))
    return Z_all, logP_all


def exchange_carries(Z, logP, group=None):
    """All-gather every rank's slice summary given as two tensors: Z (b, h, p, n) fp32,
    logP (b, h) fp32.  Returns (Z_all (world, b, h, p, n), logP_all (world, b, h))."""
    b, h, p, n = Z.shape
    buf, Zv, lv = summary_buffer(b, h, p, n, Z.device)
    Zv.copy_(Z)
    lv.copy_(logP)
    return exchange_summaries(buf, (b, h, p, n), group)


def carry_in_state(Z_all, logP_all, rank):
    """The state entering `rank`'s slice: sum_{j<rank} exp(sum_{j<k<rank} logP_k) * Z_j.
    Plain torch, any device; the CUDA fix-up kernel computes the same thing internally."""
    s_in = torch.zeros_like(Z_all[0])
    logw = torch.zeros_like(logP_all[0])
    for j in range(rank - 1, -1, -1):
        s_in = s_in + torch.exp(logw)[..., None, None] * Z_all[j]
        logw = logw + logP_all[j]
    return s_in


def seqpar_state_path_fwd(dt, A, B, x, chunk_size, out_dtype, dt_bias=None, dt_softplus=False,
                          dt_limit=(0.0, float("inf")), initial_states=None, group=None):
    """Sequence-parallel form of `_state_path_fwd`: chunk cumsum, local scan, exchange and fix-up
    from this rank's slice of the raw dt.  Returns (dA_cumsum, dt_out, out, final) for the slice."""
    from ._ext import C
    from .kernels.state_path import _state_path_fwd
    rank = dist.get_rank(group)
    init = initial_states if rank == 0 else None
    batch, _, nheads, headdim = x.shape
    dstate = B.shape[-1]
    buf, Z, logP = summary_buffer(batch, nheads, headdim, dstate, x.device)
    dA_cumsum, dt_out, out, _ = _state_path_fwd(dt, A, B, x, chunk_size, out_dtype, dt_bias=dt_bias,
                                                dt_softplus=dt_softplus, dt_limit=dt_limit, initial_states=init,
                                                final_states=Z)
    dA_last = dA_cumsum[:, :, :, -1]
    torch.sum(dA_last, dim=-1, out=logP)
    Z_all, logP_all = exchange_summaries(buf, (batch, nheads, headdim, dstate), group)
    if rank > 0:
        C.seqpar_fixup(Z_all, logP_all, rank, dA_last, out, Z)      # Z becomes the state leaving the slice
    return dA_cumsum, dt_out, out, Z


def seqpar_fused_state_fwd(B, x, dt, dA_cumsum, out_dtype, initial_states=None, group=None):
    """Sequence-parallel form of the fused entry point.  Arguments are this rank's slice
    (dt, dA_cumsum from `_chunk_cumsum_fwd` on the slice); `initial_states` is honoured on rank
    0 only.  Returns (out, final) for the slice; `final` of the LAST rank is the sequence's
    final state, and every rank's `final` is the state leaving its slice."""
    from ._ext import C
    from .kernels._fused import _fused_chunk_state_state_passing_fwd as fused
    rank = dist.get_rank(group)
    init = initial_states if rank == 0 else None
    batch, _, nheads, headdim = x.shape
    dstate = B.shape[-1]
    # the local scan leaves its final state directly in the buffer that is exchanged
    buf, Z, logP = summary_buffer(batch, nheads, headdim, dstate, x.device)
    out, _ = fused(B, x, dt, dA_cumsum, out_dtype, initial_states=init, final_states=Z)
    dA_last = dA_cumsum[:, :, :, -1]
    torch.sum(dA_last, dim=-1, out=logP)
    Z_all, logP_all = exchange_summaries(buf, (batch, nheads, headdim, dstate), group)
    if rank > 0:
        C.seqpar_fixup(Z_all, logP_all, rank, dA_last, out, Z)      # Z becomes the state leaving the slice
    return out, Z
