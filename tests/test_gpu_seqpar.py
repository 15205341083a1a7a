"""Sequence-parallel state path on the GPU: the fix-up kernel with the ranks emulated one after
another on one device, and (when the box has two or more GPUs) the real thing over NCCL."""
import os
import socket

import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(device, b, l, h, g, seed, dtype=torch.bfloat16):
    return {k: v.to(device) for k, v in O.make_inputs(b, l, h, 64, g, 128, dtype=dtype, seed=seed).items()}


@pytest.mark.parametrize("world,l,L,with_init", [(2, 2048, 256, False), (4, 3000, 128, True), (8, 4096, 64, False)])
def test_fixup_kernel_with_emulated_ranks(cuda_device, world, l, L, with_init):
    from mamba_fused_minimal_b200 import parallel as P
    from mamba_fused_minimal_b200._ext import C
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    b, h, g = 2, 4, 1
    d = _inputs(cuda_device, b, l, h, g, seed=17)
    init = torch.randn(b, h, 64, 128, device=cuda_device) if with_init else None
    dA_f, dt_f = _chunk_cumsum_fwd(d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    out_f, fin_f = fused(d["B"], d["x"], dt_f, dA_f, torch.bfloat16, initial_states=init)

    locals_ = []
    for r in range(world):
        s0, s1 = P.shard_sequence(l, L, world, r)
        dA, dt = _chunk_cumsum_fwd(d["dt"][:, s0:s1], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
        out, Z = fused(d["B"][:, s0:s1], d["x"][:, s0:s1], dt, dA, torch.bfloat16,
                       initial_states=init if r == 0 else None)
        locals_.append((s0 // L, dA[:, :, :, -1], out, Z))
    Z_all = torch.stack([t[3] for t in locals_]).contiguous()
    logP_all = torch.stack([t[1].sum(-1) for t in locals_]).contiguous()
    for r, (c0, dA_last, out, Z) in enumerate(locals_):
        if r > 0:
            C.seqpar_fixup(Z_all, logP_all, r, dA_last, out, Z)
        torch.cuda.synchronize()
        ref = out_f[:, c0:c0 + out.shape[1]].float()
        scale = out_f.float().abs().max().item()
        # passed states: re-rounded once more where a carry was added, so one bf16 ulp apart at most
        torch.testing.assert_close(out.float() / scale, ref / scale, atol=1e-2, rtol=1e-2)
        nxt = out_f[:, c0 + out.shape[1]].float() if c0 + out.shape[1] < out_f.shape[1] else fin_f
        tol = 1e-2 if nxt is not fin_f else 1e-3          # a bf16 neighbour vs the fp32 final state
        err = (Z - nxt).abs().max().item() / nxt.abs().max().item()
        assert err <= tol, (r, err)
    # the kernel's carried state against the plain-torch composition of the same summaries:
    # final_r - Z_r = exp(logP_r) * S_in,r
    for r, (c0, dA_last, out, Z) in enumerate(locals_):
        s_in = P.carry_in_state(Z_all, logP_all, r)
        want = Z_all[r] + torch.exp(logP_all[r])[..., None, None] * s_in
        err = (Z - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
        assert err <= 1e-5, (r, err)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _nccl_rank(rank, world, port, q):
    try:
        import torch.distributed as dist
        from mamba_fused_minimal_b200 import parallel as P
        from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
        from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                device_id=dev)
        b, l, h, g, L = 1, 8192, 8, 1, 256
        d = _inputs(dev, b, l, h, g, seed=23)
        dA_f, dt_f = _chunk_cumsum_fwd(d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
        out_f, fin_f = fused(d["B"], d["x"], dt_f, dA_f, torch.bfloat16)
        s0, s1 = P.shard_sequence(l, L, world, rank)
        dA, dt = _chunk_cumsum_fwd(d["dt"][:, s0:s1], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
        out, fin = P.seqpar_fused_state_fwd(d["B"][:, s0:s1], d["x"][:, s0:s1], dt, dA, torch.bfloat16)
        torch.cuda.synchronize()
        c0 = s0 // L
        scale = out_f.float().abs().max().item()
        err_out = ((out.float() - out_f[:, c0:c0 + out.shape[1]].float()).abs().max() / scale).item()
        err_fin = None
        if rank == world - 1:
            err_fin = ((fin - fin_f).abs().max() / fin_f.abs().max()).item()
        q.put((rank, err_out, err_fin, None))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        q.put((rank, None, None, repr(e)))


def test_sequence_parallel_over_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, err_out, err_fin, exc in results:
        assert exc is None, f"rank {rank}: {exc}"
        assert err_out <= 1e-2, (rank, err_out)
        if err_fin is not None:
            assert err_fin <= 1e-3, err_fin
