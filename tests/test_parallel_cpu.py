"""Host-side logic of the multi-GPU layer on CPU ranks (gloo): the sharding helpers, and the
sequence-parallel carry protocol (all-gather of slice summaries, carry-in composition) checked
against the oracle run on the whole sequence.  The per-slice math is done by the oracle here,
since the CUDA kernels need a GPU; what is under test is the exchange and the composition."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mamba_fused_minimal_b200 import parallel as P
from oracle import ssd_oracle as O


def test_shard_ranges_cover_everything():
    for n, world in [(80, 8), (80, 3), (7, 8), (128, 4)]:
        got = []
        for r in range(world):
            a, b = P.shard_range(n, world, r)
            got += list(range(a, b))
        assert got == list(range(n))


def test_shard_heads_keeps_groups_whole():
    (h0, h1), (g0, g1) = P.shard_heads(128, 8, 8, 3)
    assert (h0, h1) == (48, 64) and (g0, g1) == (3, 4)
    (h0, h1), (g0, g1) = P.shard_heads(80, 1, 8, 7)
    assert (h0, h1) == (70, 80) and (g0, g1) == (0, 1)


def test_shard_sequence_is_chunk_aligned():
    assert P.shard_sequence(1048576, 256, 8, 1) == (131072, 262144)
    spans = [P.shard_sequence(1000, 256, 3, r) for r in range(3)]
    assert spans == [(0, 512), (512, 768), (768, 1000)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, seqlen, with_init, result_queue):
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        torch.set_num_threads(1)
        b, h, p, g, n, L = 2, 4, 16, 2, 8, 32
        inp = O.make_inputs(b, seqlen, h, p, g, n, dtype=torch.float32, seed=3)
        gen = torch.Generator().manual_seed(9)
        init = torch.randn(b, h, p, n, generator=gen) if with_init else None
        # the truth: one pass over the whole sequence
        dA_f, dt_f = O.chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
        out_f, fin_f = O.fused_state_fwd(inp["B"], inp["x"], dt_f, dA_f, torch.float32, initial_states=init)
        # this rank's slice
        s0, s1 = P.shard_sequence(seqlen, L, world, rank)
        c0 = s0 // L
        sl = slice(s0, s1)
        dA, dt = O.chunk_cumsum_fwd(inp["dt"][:, sl], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
        out0, Z = O.fused_state_fwd(inp["B"][:, sl], inp["x"][:, sl], dt, dA, torch.float32,
                                    initial_states=init if rank == 0 else None)
        dA_last = dA[:, :, :, -1]
        Z_all, logP_all = P.exchange_carries(Z, dA_last.sum(-1))
        assert Z_all.shape == (world, b, h, p, n) and torch.equal(Z_all[rank], Z)
        s_in = P.carry_in_state(Z_all, logP_all, rank)
        cum = torch.cumsum(dA_last, dim=-1) - dA_last                      # exclusive, b h c
        out = out0 + torch.exp(cum).permute(0, 2, 1)[..., None, None] * s_in[:, None]
        fin = Z + torch.exp(dA_last.sum(-1))[..., None, None] * s_in
        nloc = out.shape[1]
        err_out = (out - out_f[:, c0:c0 + nloc]).abs().max().item() / out_f.abs().max().item()
        # the state leaving this slice equals the state entering the next one in the full run
        nxt = out_f[:, c0 + nloc] if c0 + nloc < out_f.shape[1] else fin_f
        err_fin = (fin - nxt).abs().max().item() / fin_f.abs().max().item()
        result_queue.put((rank, err_out, err_fin))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # surface the failure to the parent instead of hanging it
        result_queue.put((rank, repr(e), None))


@pytest.mark.parametrize("world,seqlen,with_init", [(2, 256, False), (3, 330, True)])
def test_sequence_parallel_protocol_on_cpu_ranks(world, seqlen, with_init):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, seqlen, with_init, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for pr in procs:
        pr.join(timeout=60)
    for rank, err_out, err_fin in results:
        assert err_fin is not None, f"rank {rank} failed: {err_out}"
        assert err_out < 1e-5 and err_fin < 1e-5, (rank, err_out, err_fin)
