"""Seeded test inputs: `generate_dummy_data` as in the reference (kernels/rand_data.py:4-26;
seed 42, every tensor in one dtype, A in (-1, 0], dt in [0.5, 1), dt_bias in [-0.25, 0.25)),
and `generate_benchmark_data` with the value distributions of the benchmark configurations."""
import math

import torch


def generate_dummy_data(n_groups=1, dstate=128, nheads=80, headdim=64, seq_len=2048, dtype=torch.bfloat16,
                        device=torch.device("cuda"), chunk_size=256, batch_size=1):
    torch.manual_seed(42)
    x = torch.randn((batch_size, seq_len, nheads, headdim), dtype=dtype, device=device)
    A = torch.rand((nheads,), dtype=dtype, device=device) * -1
    B = torch.randn((batch_size, seq_len, n_groups, dstate), dtype=dtype, device=device)
    C = torch.randn((batch_size, seq_len, n_groups, dstate), dtype=dtype, device=device)
    D = torch.randn((nheads,), dtype=dtype, device=device)
    dt = torch.rand((batch_size, seq_len, nheads), dtype=dtype, device=device) * 0.5 + 0.5
    dt_bias = torch.rand((nheads,), dtype=dtype, device=device) * 0.5 - 0.25
    return x, A, B, C, D, dt, dt_bias


def generate_benchmark_data(batch, seqlen, nheads, headdim, ngroups, dstate, dtype=torch.bfloat16,
                            device=torch.device("cuda"), seed=0):
    """x, B, C, D ~ N(0,1); dt ~ N(0,1) (softplus and bias are applied by the cumsum step);
    dt_bias = inverse softplus of U[1e-3, 1e-1]; A = -exp(U[0, ln 16]).  Drawn on `device`.
    Returns a dict."""
    gen = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((batch, seqlen, nheads, headdim), generator=gen, device=device, dtype=torch.float32).to(dtype)
    dt = torch.randn((batch, seqlen, nheads), generator=gen, device=device)
    d0 = torch.rand((nheads,), generator=gen, device=device) * (1e-1 - 1e-3) + 1e-3
    dt_bias = d0 + torch.log(-torch.expm1(-d0))
    A = -torch.exp(torch.rand((nheads,), generator=gen, device=device) * math.log(16.0))
    B = torch.randn((batch, seqlen, ngroups, dstate), generator=gen, device=device).to(dtype)
    C = torch.randn((batch, seqlen, ngroups, dstate), generator=gen, device=device).to(dtype)
    D = torch.randn((nheads,), generator=gen, device=device)
    return dict(x=x, dt=dt, dt_bias=dt_bias, A=A, B=B, C=C, D=D)
