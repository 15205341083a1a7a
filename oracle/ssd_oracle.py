"""CPU oracle for the Mamba2 SSD forward hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch on the CPU, the arithmetic of the reference
repository's Triton kernels (RishiAstra/mamba-fused-minimal), keeping the reference's
rounding points (where a value is cast to the input dtype before a dot product, where the
running state stays in fp32, where an output is rounded on store).  It is the checker the
CUDA kernels are compared with; it is never the product path.  Only the test-suite, the
smoke check and the benchmark's CPU-baseline leg may import it.

Parity pin: every function here is compared, in tests/test_oracle_golden.py, with outputs
of the reference's own kernels executed under the Triton interpreter
(tests/golden/make_golden.py generated the committed fixtures from the reference sources),
and with fixtures produced by the reference's compiled Triton kernels on a B200 for the
16-bit input types, which the interpreter cannot execute.

Reference lines followed (paths inside the reference project):
  chunk_cumsum_fwd      kernels/ssd_chunk_state.py:65-79,176-199
  chunk_state_fwd       kernels/ssd_chunk_state.py:134-173,202-232
  state_passing_fwd     kernels/ssd_state_passing.py:61-84,87-115
  fused_state_fwd       kernels/fused_concurrent.py:255-331 / kernels/fused_globalbar.py:201-266
  bmm_chunk_fwd         kernels/ssd_bmm.py:64-87,89-134
  chunk_scan_fwd        kernels/ssd_chunk_scan.py:83-169,172-221
  combined_fwd          main.py:60-74
  ssd_sequential        independent per-token recurrence (no reference counterpart); second opinion
"""
import math

import torch
import torch.nn.functional as F


def _nchunks(seqlen, chunk_size):
    return (seqlen + chunk_size - 1) // chunk_size


def _pad_seq(t, chunk_size, dim=1):
    """Zero-pad dimension `dim` (the sequence) to a whole number of chunks."""
    seqlen = t.shape[dim]
    pad = _nchunks(seqlen, chunk_size) * chunk_size - seqlen
    if pad == 0:
        return t
    shape = list(t.shape)
    shape[dim] = pad
    return torch.cat([t, torch.zeros(shape, dtype=t.dtype)], dim=dim)


LOG2E_F32 = 1.4426950408889634


def _exp(x, impl="exact"):
    """exp(x) in fp32.  "exact": torch.exp (what the Triton interpreter computes).  "ex2":
    2^(fl32(x * log2 e)), the form `tl.exp` compiles to on NVIDIA GPUs -- the rounding of the
    product to fp32 is what distinguishes the two (up to a few 1e-6 relative for |x| ~ 100),
    enough to flip the 16-bit rounding of a scaled B element now and then."""
    x = x.float()
    if impl == "exact":
        return torch.exp(x)
    assert impl == "ex2"
    return torch.exp2(x * torch.tensor(LOG2E_F32, dtype=torch.float32))


def softplus_ref(x):
    """kernels/softplus.py:8-10 (Triton >= 3 form): log(exp(x) + 1)."""
    return torch.log(torch.exp(x) + 1.0)


def chunk_cumsum_fwd(dt, A, chunk_size, dt_bias=None, dt_softplus=False,
                     dt_limit=(0.0, float("inf"))):
    """Returns (dA_cumsum, dt_out), both (batch, nheads, nchunks, chunk_size) fp32.

    dt (batch, seqlen, nheads); A (nheads,); dt_bias (nheads,) or None.
    Order of operations as in kernels/ssd_chunk_state.py:65-78: add bias, softplus where
    dt <= 20, clamp to dt_limit, zero past seqlen, multiply by A, inclusive cumsum.
    """
    batch, seqlen, nheads = dt.shape
    assert A.shape == (nheads,)
    nchunks = _nchunks(seqlen, chunk_size)
    d = dt.float()
    if dt_bias is not None:
        assert dt_bias.shape == (nheads,)
        d = d + dt_bias.float()[None, None, :]
    if dt_softplus:
        d = torch.where(d <= 20.0, softplus_ref(d), d)
    d = torch.clamp(d, min=dt_limit[0], max=dt_limit[1])
    d = _pad_seq(d, chunk_size)                       # positions past seqlen hold dt = 0
    d = d.view(batch, nchunks, chunk_size, nheads).permute(0, 3, 1, 2).contiguous()
    dA = d * A.float()[None, :, None, None]
    dA_cumsum = torch.cumsum(dA, dim=-1, dtype=torch.float32)
    return dA_cumsum, d


def _chunked(t, chunk_size):
    """(batch, seqlen, ...) -> (batch, nchunks, chunk_size, ...), zero padded."""
    t = _pad_seq(t, chunk_size)
    b, lp = t.shape[:2]
    return t.view(b, lp // chunk_size, chunk_size, *t.shape[2:])


def chunk_state_fwd(B, x, dt, dA_cumsum, seq_idx=None, states=None, states_in_fp32=True,
                    clamp_decay=True, exp_impl="exact"):
    """Per-chunk states (batch, nchunks, nheads, headdim, dstate).

    states[p, n] = sum_k x[k, p] * cast(B[k, n] * exp(min(dA_last - dA_k, 0)) * dt_k),
    the cast going to x's dtype before the dot and the sum running in fp32
    (kernels/ssd_chunk_state.py:153-159).  `clamp_decay=False` gives the fused kernels'
    unclamped exponent (kernels/fused_concurrent.py:119).
    """
    batch, seqlen, nheads, headdim = x.shape
    _, _, nchunks, chunk_size = dt.shape
    _, _, ngroups, dstate = B.shape
    assert nheads % ngroups == 0
    assert B.shape == (batch, seqlen, ngroups, dstate)
    assert dt.shape == (batch, nheads, nchunks, chunk_size)
    assert dA_cumsum.shape == dt.shape
    ratio = nheads // ngroups
    xc = _chunked(x, chunk_size)                              # b c k h p
    Bc = _chunked(B, chunk_size).float()                      # b c k g n
    Bc = Bc.repeat_interleave(ratio, dim=3)                   # b c k h n
    dA = dA_cumsum.float()
    expo = dA[..., -1:] - dA                                  # b h c k
    if clamp_decay:
        expo = torch.clamp(expo, max=0.0)
    scale = _exp(expo, exp_impl) * dt.float()                 # b h c k
    if seq_idx is not None:
        assert seq_idx.shape == (batch, seqlen)
        sic = _chunked(seq_idx.to(torch.int64) + 1, chunk_size) - 1     # pad = -1
        limit = torch.clamp(seqlen - torch.arange(nchunks) * chunk_size, max=chunk_size)
        last = torch.gather(sic, 2, (limit - 1).view(1, nchunks, 1).expand(batch, -1, 1))
        same = (sic == last)                                  # b c k
        scale = torch.where(same[:, None], scale, torch.zeros_like(scale))
    bs = (Bc * scale.permute(0, 2, 3, 1)[..., None]).to(x.dtype)   # rounding point
    out = torch.einsum("bckhp,bckhn->bchpn", xc.float(), bs.float())
    out_dtype = torch.float32 if states_in_fp32 else B.dtype
    if states is not None:
        assert states.shape == (batch, nchunks, nheads, headdim, dstate)
        states.copy_(out.to(states.dtype))
        return states
    return out.to(out_dtype)


def state_passing_fwd(states, dA_chunk_cumsum, initial_states=None, seq_idx=None,
                      chunk_size=None, out_dtype=None, exp_impl="exact"):
    """Exclusive scan of the chunk states (kernels/ssd_state_passing.py:61-84).

    states (batch, nchunks, nheads, dim); dA_chunk_cumsum (batch, nheads, nchunks).
    Returns out (batch, nchunks, nheads, dim) in out_dtype, final_states (batch, nheads, dim)
    fp32.  The running state stays fp32; only the store rounds.
    """
    batch, nchunks, nheads, dim = states.shape
    assert dA_chunk_cumsum.shape == (batch, nheads, nchunks)
    out_dtype = states.dtype if out_dtype is None else out_dtype
    out = torch.empty(batch, nchunks, nheads, dim, dtype=out_dtype)
    if initial_states is None:
        s = torch.zeros(batch, nheads, dim, dtype=torch.float32)
    else:
        assert initial_states.shape == (batch, nheads, dim)
        s = initial_states.float().clone()
    if seq_idx is not None:
        assert chunk_size is not None
        seqlen = seq_idx.shape[-1]
        prev = torch.zeros(batch, dtype=torch.int64)
    for c in range(nchunks):
        out[:, c] = s.to(out_dtype)
        scale = _exp(dA_chunk_cumsum[:, :, c], exp_impl)                 # b h
        if seq_idx is not None:
            new = seq_idx[:, min((c + 1) * chunk_size, seqlen) - 1].to(torch.int64)
            scale = torch.where((new == prev)[:, None], scale, torch.zeros_like(scale))
            prev = new
        s = scale[..., None] * s + states[:, c].float()
    return out, s


def fused_state_fwd(B, x, dt, dA_cumsum, out_dtype, initial_states=None, seq_idx=None,
                    states=None, states_in_fp32=True, exp_impl="exact"):
    """What both fused entry points return: (out (b,c,h,p,n) out_dtype, final (b,h,p,n) fp32).

    Composition of the two functions above (that composition is what the reference's own
    check asserts, main.py:174-182).  initial_states is (b,h,p,n) here
    (kernels/fused_concurrent.py:277).
    """
    st = chunk_state_fwd(B, x, dt, dA_cumsum, seq_idx=seq_idx, states=states,
                         states_in_fp32=states_in_fp32, exp_impl=exp_impl)
    b, c, h, p, n = st.shape
    chunk_size = dt.shape[-1]
    init = None if initial_states is None else initial_states.reshape(b, h, p * n)
    out, fin = state_passing_fwd(st.reshape(b, c, h, p * n), dA_cumsum[:, :, :, -1],
                                 initial_states=init, seq_idx=seq_idx, chunk_size=chunk_size,
                                 out_dtype=st.dtype if out_dtype is None else out_dtype,
                                 exp_impl=exp_impl)
    return out.view(b, c, h, p, n), fin.view(b, h, p, n)


def bmm_chunk_fwd(a, b, chunk_size, seq_idx=None, causal=False, output_dtype=None):
    """out[b,c,(g,)i,j] = sum_k a[i,k] b[j,k] inside each chunk (kernels/ssd_bmm.py:64-87).

    With causal=True the reference leaves tiles strictly above the diagonal unwritten; the
    oracle fills the full matrix, so compare only the lower triangle in that mode.
    """
    has_groups = a.dim() == 4
    if not has_groups:
        a = a[:, :, None]
        b = b[:, :, None]
    batch, seqlen, ngroups, k = a.shape
    assert b.shape == a.shape
    if a.dtype == torch.bfloat16 or b.dtype == torch.bfloat16:
        dot = torch.bfloat16
    elif a.dtype == torch.float16 or b.dtype == torch.float16:
        dot = torch.float16
    else:
        dot = torch.float32
    ac = _chunked(a.to(dot), chunk_size).float()
    bc = _chunked(b.to(dot), chunk_size).float()
    out = torch.einsum("bcigk,bcjgk->bcgij", ac, bc)
    if seq_idx is not None:
        sm = _chunked(seq_idx.to(torch.int64) + 2, chunk_size) - 2          # pad = -2
        sn = _chunked(seq_idx.to(torch.int64) + 3, chunk_size) - 3          # pad = -3
        out = torch.where((sm[:, :, :, None] == sn[:, :, None, :])[:, :, None], out,
                          torch.zeros_like(out))
    out = out.to(a.dtype if output_dtype is None else output_dtype)
    return out if has_groups else out[:, :, 0]


def chunk_scan_fwd(cb, x, dt, dA_cumsum, C, states, D=None, z=None, seq_idx=None,
                   exp_impl="exact"):
    """Returns (out, out_x) (kernels/ssd_chunk_scan.py:83-169).

    out[m] = exp(dA_m) * C[m] . cast(prev_state)  +  sum_{k<=m} cast(cb[m,k] *
             exp(min(dA_m - dA_k, 0)) * dt_k) * x[k]  +  D * x[m],   then the z gate.
    Casts go to C's dtype for prev_state and x's dtype for the cb term; sums are fp32.
    """
    batch, seqlen, nheads, headdim = x.shape
    _, _, nchunks, chunk_size = dt.shape
    _, _, ngroups, dstate = C.shape
    assert C.shape == (batch, seqlen, ngroups, dstate)
    assert cb.shape == (batch, nchunks, ngroups, chunk_size, chunk_size)
    assert states.shape == (batch, nchunks, nheads, headdim, dstate)
    ratio = nheads // ngroups
    L = chunk_size
    xc = _chunked(x, L)                                                # b c k h p
    Cc = _chunked(C, L).repeat_interleave(ratio, dim=3)                # b c m h n
    dA = dA_cumsum.float()                                             # b h c L
    scale_m = _exp(dA, exp_impl)                                       # b h c m
    if seq_idx is not None:
        sic = _chunked(seq_idx.to(torch.int64) + 1, L) - 1             # b c m, pad -1
        prev = torch.zeros(batch, nchunks, dtype=torch.int64)
        if nchunks > 1:
            prev[:, 1:] = seq_idx[:, L - 1:(nchunks - 1) * L:L].to(torch.int64)
        same = sic == prev[:, :, None]
        scale_m = torch.where(same[:, None], scale_m, torch.zeros_like(scale_m))
    prev_states = states.to(C.dtype).float()                           # b c h p n
    acc = torch.einsum("bcmhn,bchpn->bcmhp", Cc.float(), prev_states)
    acc = acc * scale_m.permute(0, 2, 3, 1)[..., None]
    cbh = cb.float().repeat_interleave(ratio, dim=2)                   # b c h m k
    seg = torch.clamp(dA[..., :, None] - dA[..., None, :], max=0.0)    # b h c m k
    w = cbh * _exp(seg, exp_impl).permute(0, 2, 1, 3, 4)
    w = w * dt.float().permute(0, 2, 1, 3)[:, :, :, None, :]
    causal = torch.tril(torch.ones(L, L, dtype=torch.bool))
    w = torch.where(causal, w, torch.zeros_like(w)).to(x.dtype)        # rounding point
    acc = acc + torch.einsum("bchmk,bckhp->bcmhp", w.float(), xc.float())
    if D is not None:
        Df = D.float()
        Df = Df[None, None, None, :, None] if D.dim() == 1 else Df[None, None, None]
        acc = acc + xc.float() * Df
    acc = acc.reshape(batch, nchunks * L, nheads, headdim)[:, :seqlen]
    out_x = None
    if z is not None:
        out_x = acc.to(x.dtype)
        zf = z.float()
        acc = acc * (zf * torch.sigmoid(zf))
    return acc.to(x.dtype), out_x


def combined_fwd(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None,
                 initial_states=None, dt_softplus=False, dt_limit=(0.0, float("inf")),
                 exp_impl="exact"):
    """The reference's unfused pipeline, main.py:60-74.  Returns the same 6-tuple
    (out, out_x, dt, dA_cumsum, states, final_states)."""
    dA_cumsum, dt_out = chunk_cumsum_fwd(dt, A, chunk_size, dt_bias=dt_bias,
                                         dt_softplus=dt_softplus, dt_limit=dt_limit)
    states, final_states = fused_state_fwd(B, x, dt_out, dA_cumsum, C.dtype,
                                           initial_states=initial_states, exp_impl=exp_impl)
    CB = bmm_chunk_fwd(C, B, chunk_size, output_dtype=torch.float32)
    out, out_x = chunk_scan_fwd(CB, x, dt_out, dA_cumsum, C, states, D=D, z=z,
                                exp_impl=exp_impl)
    return out, out_x, dt_out, dA_cumsum, states, final_states


def hot_path_fwd(x, dt, A, B, chunk_size, dt_bias=None, dt_softplus=False,
                 dt_limit=(0.0, float("inf")), out_dtype=None, initial_states=None,
                 exp_impl="exact"):
    """cumsum -> chunk state -> state passing: the timed path.  Returns
    (dA_cumsum, dt_out, out, final_states)."""
    dA_cumsum, dt_out = chunk_cumsum_fwd(dt, A, chunk_size, dt_bias=dt_bias,
                                         dt_softplus=dt_softplus, dt_limit=dt_limit)
    out, fin = fused_state_fwd(B, x, dt_out, dA_cumsum,
                               B.dtype if out_dtype is None else out_dtype,
                               initial_states=initial_states, exp_impl=exp_impl)
    return dA_cumsum, dt_out, out, fin


def ssd_sequential(x, dt, A, B, C, D=None, dt_bias=None, dt_softplus=False,
                   dt_limit=(0.0, float("inf")), initial_states=None):
    """Token-by-token recurrence in fp64: h_t = exp(dt_t A) h_{t-1} + dt_t x_t (x) B_t,
    y_t = C_t . h_t + D x_t.  Returns (y (b,l,h,p) fp64, final state (b,h,p,n) fp64).
    Shares no code with the chunked functions above."""
    batch, seqlen, nheads, headdim = x.shape
    ngroups, dstate = B.shape[2:]
    ratio = nheads // ngroups
    d = dt.double()
    if dt_bias is not None:
        d = d + dt_bias.double()
    if dt_softplus:
        d = torch.where(d <= 20.0, torch.log1p(torch.exp(d)), d)
    d = torch.clamp(d, dt_limit[0], dt_limit[1])
    Bh = B.double().repeat_interleave(ratio, dim=2)
    Ch = C.double().repeat_interleave(ratio, dim=2)
    h = (torch.zeros(batch, nheads, headdim, dstate, dtype=torch.float64)
         if initial_states is None else initial_states.double().clone())
    y = torch.empty(batch, seqlen, nheads, headdim, dtype=torch.float64)
    Ad = A.double()
    for t in range(seqlen):
        decay = torch.exp(d[:, t] * Ad)                                   # b h
        h = decay[..., None, None] * h + (d[:, t, :, None] * x[:, t].double())[..., None] \
            * Bh[:, t, :, None, :]
        y[:, t] = torch.einsum("bhpn,bhn->bhp", h, Ch[:, t])
        if D is not None:
            Dd = D.double()
            y[:, t] += x[:, t].double() * (Dd[None, :, None] if D.dim() == 1 else Dd[None])
    return y, h


# ----------------------------------------------------------------------------------------
# Seeded synthetic inputs

def make_inputs(batch, seqlen, nheads, headdim, ngroups, dstate, dtype=torch.float32, seed=0,
                device="cpu"):
    """Inputs with the value distributions of the benchmark configurations:
    x, B, C, D ~ N(0,1); dt = N(0,1) (softplus and bias applied by the cumsum step);
    dt_bias = inverse-softplus(U[1e-3, 1e-1]); A = -exp(U[0, ln 16]).
    Generation order is fixed so a seed names one data set."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(batch, seqlen, nheads, headdim, generator=gen).to(dtype)
    dt = torch.randn(batch, seqlen, nheads, generator=gen)
    d0 = torch.rand(nheads, generator=gen) * (1e-1 - 1e-3) + 1e-3
    dt_bias = d0 + torch.log(-torch.expm1(-d0))
    A = -torch.exp(torch.rand(nheads, generator=gen) * math.log(16.0))
    B = torch.randn(batch, seqlen, ngroups, dstate, generator=gen).to(dtype)
    C = torch.randn(batch, seqlen, ngroups, dstate, generator=gen).to(dtype)
    D = torch.randn(nheads, generator=gen)
    out = dict(x=x, dt=dt, dt_bias=dt_bias, A=A, B=B, C=C, D=D)
    return {k: v.to(device) for k, v in out.items()}


def make_inputs_reference_style(batch=1, seqlen=2048, nheads=80, headdim=64, ngroups=1,
                                dstate=128, dtype=torch.bfloat16, seed=42):
    """Inputs distributed as the reference's own generator draws them
    (kernels/rand_data.py:17-24): every tensor in `dtype`, A in (-1,0], dt in [0.5,1),
    dt_bias in [-0.25,0.25).  Drawn on the CPU generator, so the values differ from a CUDA
    draw with the same seed; the distributions are the same."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(batch, seqlen, nheads, headdim, generator=gen).to(dtype)
    A = (torch.rand(nheads, generator=gen) * -1).to(dtype)
    B = torch.randn(batch, seqlen, ngroups, dstate, generator=gen).to(dtype)
    C = torch.randn(batch, seqlen, ngroups, dstate, generator=gen).to(dtype)
    D = torch.randn(nheads, generator=gen).to(dtype)
    dt = (torch.rand(batch, seqlen, nheads, generator=gen) * 0.5 + 0.5).to(dtype)
    dt_bias = (torch.rand(nheads, generator=gen) * 0.5 - 0.25).to(dtype)
    return dict(x=x, A=A, B=B, C=C, D=D, dt=dt, dt_bias=dt_bias)
