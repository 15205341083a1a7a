"""Parity of the CUDA path (Python shims -> C++ front end -> C ABI -> sm_100a kernels) with
the CPU oracle and with the reference's own outputs stored in tests/golden/.

Tolerances (the ones the build is held to): fp32 tensors within 1e-3 of the tensor's largest
magnitude (max|a-b| / max|b|); 16-bit outputs within atol = rtol = 1e-2 (in units of the
tensor's largest magnitude for atol).  Most cases land orders of magnitude inside these."""
import math

import pytest
import torch

from conftest import golden_names, load_golden, rel_err
from oracle import ssd_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("both_layouts")]

FP32_TOL = 1e-3


def _shims():
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent
    from mamba_fused_minimal_b200.kernels.fused_globalbar import _fused_chunk_state_state_passing_fwd_globalbar
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _chunk_scan_fwd
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd, _chunk_state_fwd
    from mamba_fused_minimal_b200.kernels.ssd_state_passing import _state_passing_fwd
    return dict(cumsum=_chunk_cumsum_fwd, chunk_state=_chunk_state_fwd, state_passing=_state_passing_fwd,
                fused_c=_fused_chunk_state_state_passing_fwd_concurrent,
                fused_g=_fused_chunk_state_state_passing_fwd_globalbar, bmm=_bmm_chunk_fwd,
                chunk_scan=_chunk_scan_fwd)


def _dev(d, device):
    return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def assert_close16(a, b, what=""):
    """16-bit outputs: atol = rtol = 1e-2, atol in units of the tensor's largest magnitude."""
    a = a.float().cpu()
    b = b.float().cpu()
    scale = max(b.abs().max().item(), 1e-30)
    torch.testing.assert_close(a / scale, b / scale, atol=1e-2, rtol=1e-2, msg=lambda m: what + ": " + m)


def assert_close32(a, b, what="", tol=FP32_TOL):
    e = rel_err(a.cpu(), b.cpu())
    assert e <= tol, f"{what}: max|a-b|/max|b| = {e:.3e} > {tol}"
    assert torch.isfinite(a).all(), what


def assert_close_auto(a, b, what=""):
    if b.dtype == torch.float32:
        assert_close32(a, b, what)
    else:
        assert_close16(a, b, what)


def run_pipeline(S, g, device, fused=None, force_general=False):
    """The reference's pipeline (main.py:60-74) on the GPU, each intermediate returned."""
    b, l, h, p, ng, n, L = [int(v) for v in g["meta"]]
    lim = (float(g["dt_limit"][0]), float(g["dt_limit"][1]))
    sp = bool(int(g["softplus"]))
    d = _dev(g, device)
    seq_idx = d.get("seq_idx")
    dA, dt = S["cumsum"](d["dt"], d["A"], L, dt_bias=d.get("dt_bias"), dt_softplus=sp, dt_limit=lim)
    st = S["chunk_state"](d["B"], d["x"], dt, dA, seq_idx=seq_idx)
    init = d.get("init")
    if fused is None:
        passed, fin = S["state_passing"](st.reshape(b, -1, h, p * n), dA[:, :, :, -1],
                                         initial_states=None if init is None else init.reshape(b, h, p * n),
                                         seq_idx=seq_idx, chunk_size=L, out_dtype=d["C"].dtype)
        passed = passed.view(b, -1, h, p, n)
        fin = fin.view(b, h, p, n)
    else:
        passed, fin = S[fused](d["B"], d["x"], dt, dA, d["C"].dtype, initial_states=init, seq_idx=seq_idx)
    cb = S["bmm"](d["C"], d["B"], L, seq_idx=seq_idx, output_dtype=torch.float32)
    out, out_x = S["chunk_scan"](cb, d["x"], dt, dA, d["C"], passed, D=d.get("D"), z=d.get("z"), seq_idx=seq_idx)
    torch.cuda.synchronize()
    return dict(o_dA_cumsum=dA, o_dt=dt, o_states=st, o_passed=passed, o_final=fin, o_CB=cb, o_out=out,
                o_out_x=out_x)


@pytest.mark.parametrize("fused", [None, "fused_c", "fused_g"])
@pytest.mark.parametrize("name", golden_names("interp_") + golden_names("gpu_"))
def test_against_reference_golden(cuda_device, name, fused):
    """Every function against the reference's own outputs (fp32: interpreter; 16-bit: B200)."""
    g = load_golden(name)
    res = run_pipeline(_shims(), g, cuda_device, fused=fused)
    for k, v in res.items():
        if v is None:
            assert k not in g
            continue
        assert v.shape == g[k].shape, k
        assert v.dtype == g[k].dtype, k
        assert_close_auto(v, g[k], f"{name}:{k}")


CASES = [
    # b, l, h, p, g, n, L, dtype, opts
    (2, 512, 8, 64, 1, 128, 128, torch.bfloat16, {}),                        # tcgen05 path, 2 heads per CTA
    (1, 1000, 6, 64, 2, 128, 256, torch.bfloat16, dict(init=True)),          # ragged tail, 3 heads per group (1 head per CTA)
    (3, 384, 4, 64, 4, 128, 64, torch.float16, dict(init=True)),             # fp16, one head per group
    (1, 8192, 2, 64, 1, 128, 64, torch.bfloat16, {}),                        # one strip over many CTAs: chained carries
    (2, 320, 4, 32, 2, 16, 64, torch.float32, dict(init=True)),              # plain kernels, fp32
    (1, 257, 3, 48, 1, 40, 96, torch.bfloat16, dict(init=True)),             # odd sizes everywhere
    (2, 256, 4, 64, 1, 128, 128, torch.bfloat16, dict(out_fp32=True, states_buf=True)),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "b%d_l%d_h%d_p%d_g%d_n%d_L%d_%s" % (c[:7] + (str(c[7]).split(".")[-1],)))
def test_state_path_against_oracle(cuda_device, case):
    b, l, h, p, ng, n, L, dtype, opt = case
    S = _shims()
    inp = O.make_inputs(b, l, h, p, ng, n, dtype=dtype, seed=7)
    gen = torch.Generator().manual_seed(3)
    init = torch.randn(b, h, p, n, generator=gen) if opt.get("init") else None
    out_dtype = torch.float32 if opt.get("out_fp32") else dtype
    ref_dA, ref_dt = O.chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)

    d = _dev(inp, cuda_device)
    dA, dt = S["cumsum"](d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    assert_close32(dA, ref_dA, "dA_cumsum", tol=1e-5)
    assert_close32(dt, ref_dt, "dt", tol=1e-5)
    # the later stages are compared on IDENTICAL inputs: the oracle gets the dt / dA_cumsum
    # the GPU produced (two valid cumsums differ in the last bits, and the 16-bit rounding of
    # B * scale amplifies such a difference into rare one-ulp flips of a scaled element)
    dA_c, dt_c = dA.cpu(), dt.cpu()
    ref_states = O.chunk_state_fwd(inp["B"], inp["x"], dt_c, dA_c, exp_impl="ex2")
    ref_out, ref_fin = O.fused_state_fwd(inp["B"], inp["x"], dt_c, dA_c, out_dtype, initial_states=init,
                                         exp_impl="ex2")
    states = S["chunk_state"](d["B"], d["x"], dt, dA)
    assert_close32(states, ref_states, "chunk states")
    init_d = None if init is None else init.to(cuda_device)
    buf = torch.full_like(states, float("nan")) if opt.get("states_buf") else None
    for fn in ("fused_c", "fused_g"):
        out, fin = S[fn](d["B"], d["x"], dt, dA, out_dtype, initial_states=init_d, states=buf)
        assert out.dtype == out_dtype and fin.dtype == torch.float32
        assert_close_auto(out, ref_out, fn + " out")
        assert_close32(fin, ref_fin, fn + " final")
        if buf is not None:
            assert_close32(buf, ref_states, fn + " states buffer")
    # the unfused pair gives the same answer
    o2, f2 = S["state_passing"](states.reshape(b, -1, h, p * n), dA[:, :, :, -1],
                                initial_states=None if init_d is None else init_d.reshape(b, h, p * n),
                                out_dtype=out_dtype)
    assert_close_auto(o2.view_as(out), ref_out, "state_passing out")
    assert_close32(f2.view_as(fin), ref_fin, "state_passing final")
    from mamba_fused_minimal_b200._ext import C
    C.check_status(d["x"])


def test_fast_and_plain_kernels_agree(cuda_device):
    """The tcgen05 kernel and the plain CUDA-core kernels on the same inputs."""
    from mamba_fused_minimal_b200.kernels._fused import _fused_chunk_state_state_passing_fwd as fused
    S = _shims()
    inp = _dev(O.make_inputs(2, 1024, 8, 64, 2, 128, dtype=torch.bfloat16, seed=11), cuda_device)
    dA, dt = S["cumsum"](inp["dt"], inp["A"], 256, dt_bias=inp["dt_bias"], dt_softplus=True)
    o1, f1 = fused(inp["B"], inp["x"], dt, dA, torch.float32)
    o2, f2 = fused(inp["B"], inp["x"], dt, dA, torch.float32, force_general=True)
    assert_close32(o1, o2, "out", tol=1e-4)
    assert_close32(f1, f2, "final", tol=1e-4)


def test_fused_is_deterministic(cuda_device):
    S = _shims()
    inp = _dev(O.make_inputs(2, 2048, 8, 64, 1, 128, dtype=torch.bfloat16, seed=5), cuda_device)
    dA, dt = S["cumsum"](inp["dt"], inp["A"], 256, dt_bias=inp["dt_bias"], dt_softplus=True)
    o1, f1 = S["fused_c"](inp["B"], inp["x"], dt, dA, torch.bfloat16)
    o2, f2 = S["fused_c"](inp["B"], inp["x"], dt, dA, torch.bfloat16)
    assert torch.equal(o1, o2) and torch.equal(f1, f2)


def test_strided_inputs(cuda_device):
    """x, B, dt as views into larger buffers (the shape of a fused in-projection output)."""
    S = _shims()
    b, l, h, p, ng, n, L = 2, 512, 4, 64, 1, 128, 128
    inp = O.make_inputs(b, l, h, p, ng, n, dtype=torch.bfloat16, seed=9)
    width = h * p + 2 * ng * n + h
    big = torch.zeros(b, l, width + 8, dtype=torch.bfloat16)
    big[..., :h * p] = inp["x"].reshape(b, l, -1)
    big[..., h * p:h * p + ng * n] = inp["B"].reshape(b, l, -1)
    big = big.to(cuda_device)
    x = big[..., :h * p].view(b, l, h, p)
    B = big[..., h * p:h * p + ng * n].view(b, l, ng, n)
    assert not x.is_contiguous()
    d = _dev(inp, cuda_device)
    dt_big = torch.zeros(b, l, 2 * h, device=cuda_device)
    dt_big[..., ::2] = d["dt"]
    dA, dt = S["cumsum"](dt_big[..., ::2], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    ref_dA, ref_dt = O.chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
    assert_close32(dA, ref_dA, "dA", tol=1e-5)
    out, fin = S["fused_c"](B, x, dt, dA, torch.bfloat16)
    ref_out, ref_fin = O.fused_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), torch.bfloat16, exp_impl="ex2")
    assert_close16(out, ref_out, "out")
    assert_close32(fin, ref_fin, "final")


def stagewise_check(cuda_device, inp, L, D=None, z=None, init=None, fused="fused_c"):
    """All seven functions in the reference's pipeline order, each compared with the oracle
    on the inputs that stage actually received on the GPU."""
    S = _shims()
    d = _dev(inp, cuda_device)
    dev = lambda t: None if t is None else t.to(cuda_device)
    dA, dt = S["cumsum"](d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    ref_dA, ref_dt = O.chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
    assert_close32(dA, ref_dA, "dA_cumsum", tol=1e-5)
    assert_close32(dt, ref_dt, "dt", tol=1e-5)
    passed, fin = S[fused](d["B"], d["x"], dt, dA, d["C"].dtype, initial_states=dev(init))
    r_passed, r_fin = O.fused_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), inp["C"].dtype,
                                        initial_states=init, exp_impl="ex2")
    assert_close_auto(passed, r_passed, "passed states")
    assert_close32(fin, r_fin, "final states")
    cb = S["bmm"](d["C"], d["B"], L, output_dtype=torch.float32)
    assert_close32(cb, O.bmm_chunk_fwd(inp["C"], inp["B"], L, output_dtype=torch.float32), "CB", tol=1e-5)
    y, y_x = S["chunk_scan"](cb, d["x"], dt, dA, d["C"], passed, D=dev(D), z=dev(z))
    r_y, r_yx = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt.cpu(), dA.cpu(), inp["C"], passed.cpu(), D=D, z=z,
                                 exp_impl="ex2")
    assert_close_auto(y, r_y, "out")
    if z is not None:
        assert_close_auto(y_x, r_yx, "out_x")
    return dict(dA=dA, dt=dt, passed=passed, fin=fin, cb=cb, y=y)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_end_to_end_against_oracle(cuda_device, dtype):
    """All seven functions chained as in the reference's main.py, D (h,p), z gate, groups."""
    S = _shims()
    b, l, h, p, ng, n, L = 2, 600, 8, 64, 2, 128, 128
    inp = O.make_inputs(b, l, h, p, ng, n, dtype=dtype, seed=21)
    gen = torch.Generator().manual_seed(4)
    Dhp = torch.randn(h, p, generator=gen)
    z = torch.randn(b, l, h, p, generator=gen).to(dtype)
    stagewise_check(cuda_device, inp, L, D=Dhp, z=z)
    # chained: every stage fed by this library's previous stage, against the oracle's own chain.
    # Here the two cumsums differ in their last bits, which the 16-bit rounding of the scaled B
    # turns into rare one-ulp flips of a scaled element, each moving a state by up to ~0.8% of
    # one product term; the fp32 bound for chained runs is therefore 5e-3 of the tensor's max.
    ref = O.combined_fwd(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], L, D=Dhp, z=z, dt_bias=inp["dt_bias"],
                         dt_softplus=True, exp_impl="ex2")
    from mamba_fused_minimal_b200 import main as M
    d = _dev(inp, cuda_device)
    results = []
    for fn in (M._mamba_chunk_scan_combined_fwd_original, M._mamba_chunk_scan_combined_fwd_concurrent,
               M._mamba_chunk_scan_combined_fwd_globalbar):
        res = fn(d["x"], d["dt"], d["A"], d["B"], d["C"], L, D=Dhp.to(cuda_device), z=z.to(cuda_device),
                 dt_bias=d["dt_bias"], dt_softplus=True)
        results.append(res)
        for name, a, r in zip(M.TENSOR_NAMES, res, ref):
            if r.dtype == torch.float32:
                assert_close32(a, r, f"{fn.__name__}:{name}", tol=5e-3)
            else:
                assert_close16(a, r, f"{fn.__name__}:{name}")
    # the three pipelines of this library agree with each other bit for bit on the states
    for res in results[1:]:
        assert torch.equal(res[4], results[0][4]) and torch.equal(res[5], results[0][5])


def test_reference_main_check(cuda_device):
    """The reference's own acceptance run (main.py:164-190): its seed-42 bf16 inputs at
    batch 1 x 2048 x 80 heads, fused pipelines against the unfused one, its tolerance."""
    from mamba_fused_minimal_b200 import main as M
    assert M.main()


def test_seq_idx_plain_kernels(cuda_device):
    """Packed sequences: boundaries inside a chunk and on a chunk edge."""
    S = _shims()
    b, l, h, p, ng, n, L = 2, 320, 4, 32, 1, 32, 64
    inp = O.make_inputs(b, l, h, p, ng, n, dtype=torch.bfloat16, seed=13)
    seq_idx = torch.zeros(b, l, dtype=torch.int32)
    seq_idx[:, 70:] = 1
    seq_idx[:, 192:] = 2
    ref_dA, ref_dt = O.chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
    d = _dev(inp, cuda_device)
    si = seq_idx.to(cuda_device)
    dA, dt = S["cumsum"](d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    assert_close32(dA, ref_dA, "dA", tol=1e-5)
    out, fin = S["fused_c"](d["B"], d["x"], dt, dA, torch.bfloat16, seq_idx=si)
    cb = S["bmm"](d["C"], d["B"], L, seq_idx=si, output_dtype=torch.float32)
    y, _ = S["chunk_scan"](cb, d["x"], dt, dA, d["C"], out, D=d["D"], seq_idx=si)
    ref_out, ref_fin = O.fused_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), torch.bfloat16, seq_idx=seq_idx,
                                         exp_impl="ex2")
    ref_cb = O.bmm_chunk_fwd(inp["C"], inp["B"], L, seq_idx=seq_idx, output_dtype=torch.float32)
    ref_y, _ = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt.cpu(), dA.cpu(), inp["C"], out.cpu(), D=inp["D"],
                                seq_idx=seq_idx, exp_impl="ex2")
    assert_close16(out, ref_out, "out")
    assert_close32(fin, ref_fin, "final")
    assert_close32(cb, ref_cb, "cb")
    assert_close16(y, ref_y, "y")


@pytest.mark.parametrize("h,g,L", [(4, 1, 128), (3, 3, 64), (8, 2, 256)])
def test_seq_idx_tcgen05_state_path(cuda_device, h, g, L):
    """Packed sequences on the shapes the tcgen05 state kernel takes (headdim 64, dstate 128,
    16-bit inputs): boundaries inside a chunk, on a chunk edge, and a ragged last chunk; both
    the fused entry point and the per-chunk states alone."""
    S = _shims()
    b, l = 2, 5 * L + 37
    inp = O.make_inputs(b, l, h, 64, g, 128, dtype=torch.bfloat16, seed=29 + h)
    seq_idx = torch.zeros(b, l, dtype=torch.int32)
    seq_idx[:, L + 5:] = 1
    seq_idx[:, 3 * L:] = 2            # on a chunk edge
    seq_idx[1, 4 * L + 9:] = 3        # only in the second batch element
    seq_idx[:, 5 * L + 20:] = 4       # inside the ragged last chunk
    d = _dev(inp, cuda_device)
    si = seq_idx.to(cuda_device)
    dA, dt = S["cumsum"](d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    init = torch.randn(b, h, 64, 128, generator=torch.Generator().manual_seed(5))
    out, fin = S["fused_c"](d["B"], d["x"], dt, dA, torch.bfloat16, initial_states=init.to(cuda_device), seq_idx=si)
    ref_out, ref_fin = O.fused_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), torch.bfloat16, initial_states=init,
                                         seq_idx=seq_idx, exp_impl="ex2")
    assert_close16(out, ref_out, "passed states")
    assert_close32(fin, ref_fin, "final states")
    st = S["chunk_state"](d["B"], d["x"], dt, dA, seq_idx=si)
    ref_st = O.chunk_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), seq_idx=seq_idx, exp_impl="ex2")
    assert_close32(st, ref_st, "chunk states")
    # and the plain kernels on the same data
    out_p, fin_p = _fused_general(S, d, dt, dA, init.to(cuda_device), si)
    assert_close16(out, out_p.float().cpu(), "fast vs plain passed states")
    assert_close32(fin, fin_p.cpu(), "fast vs plain final states")


def _fused_general(S, d, dt, dA, init, si):
    from mamba_fused_minimal_b200.kernels._fused import _fused_chunk_state_state_passing_fwd
    return _fused_chunk_state_state_passing_fwd(d["B"], d["x"], dt, dA, torch.bfloat16, initial_states=init, seq_idx=si,
                                                force_general=True)


def test_headline_shape_properties(cuda_device):
    """Mamba2-2.7B layer shape in full (batch 8 x 4096 x 80 heads): the oracle on a slice
    (one batch element, four heads) plus size-independent properties on the whole result."""
    S = _shims()
    from mamba_fused_minimal_b200.kernels.rand_data import generate_benchmark_data
    b, l, h, p, ng, n, L = 8, 4096, 80, 64, 1, 128, 256
    d = generate_benchmark_data(b, l, h, p, ng, n, dtype=torch.bfloat16, device=cuda_device, seed=0)
    dA, dt = S["cumsum"](d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    out, fin = S["fused_c"](d["B"], d["x"], dt, dA, torch.bfloat16)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all() and torch.isfinite(fin).all()
    assert (out[:, 0] == 0).all()                      # exclusive scan starts from zero
    # slice check against the oracle: heads are independent given B
    bs, hs = 5, slice(36, 40)
    ref_dA, ref_dt = O.chunk_cumsum_fwd(d["dt"][bs:bs + 1, :, hs].cpu(), d["A"][hs].cpu(), L,
                                        dt_bias=d["dt_bias"][hs].cpu(), dt_softplus=True)
    ref_out, ref_fin = O.fused_state_fwd(d["B"][bs:bs + 1].cpu(), d["x"][bs:bs + 1, :, hs].cpu(),
                                         dt[bs:bs + 1, hs].cpu(), dA[bs:bs + 1, hs].cpu(), torch.bfloat16,
                                         exp_impl="ex2")
    assert_close32(dA[bs:bs + 1, hs], ref_dA, "dA slice", tol=1e-5)
    assert_close16(out[bs:bs + 1, :, hs], ref_out, "out slice")
    assert_close32(fin[bs:bs + 1, hs], ref_fin, "final slice")
    # linearity in x: doubling x doubles every state exactly (power of two)
    out2, fin2 = S["fused_c"](d["B"], d["x"] * 2, dt, dA, torch.bfloat16)
    assert torch.equal(fin2, fin * 2)
    assert torch.equal(out2.float(), out.float() * 2)
    # recurrence identity on the outputs themselves, in fp32 output mode:
    # S_{c+1} - exp(dA_last_c) S_c is the chunk state, which does not depend on c's history
    o32, f32 = S["fused_c"](d["B"][:1], d["x"][:1], dt[:1], dA[:1], torch.float32)
    st = S["chunk_state"](d["B"][:1], d["x"][:1], dt[:1], dA[:1])
    decay = torch.exp(dA[:1, :, :, -1]).permute(0, 2, 1)[..., None, None]      # b c h 1 1
    nxt = torch.cat([o32[:, 1:], f32[:, None]], dim=1)
    assert_close32(nxt - decay * o32, st, "recurrence identity", tol=1e-4)
    from mamba_fused_minimal_b200._ext import C
    C.check_status(d["x"])


def test_largest_shape_against_plain_kernels_on_a_slice(cuda_device):
    """The largest configuration (batch 16 x 8192, 128 heads in 8 groups): the tcgen05 kernels on the
    whole problem against the plain kernels on one batch element and one group (offsets past 2^31
    bytes, grids of thousands of tiles)."""
    from mamba_fused_minimal_b200.kernels._fused import _fused_chunk_state_state_passing_fwd
    from mamba_fused_minimal_b200.kernels.rand_data import generate_benchmark_data
    S = _shims()
    b, l, h, g, L = 16, 8192, 128, 8, 256
    d = generate_benchmark_data(b, l, h, 64, g, 128, device=cuda_device, seed=3)
    C = torch.randn_like(d["B"])
    dA, dt = S["cumsum"](d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    out, fin = S["fused_c"](d["B"], d["x"], dt, dA, torch.bfloat16)
    cb = S["bmm"](C, d["B"], L, output_dtype=torch.float32)
    Dv = torch.randn(h, device=cuda_device)
    y, _ = S["chunk_scan"](cb, d["x"], dt, dA, C, out, D=Dv)
    # slice: last batch element, last group (the far end of every tensor)
    bs, gs = b - 1, g - 1
    hs = slice(gs * (h // g), (gs + 1) * (h // g))
    xs, Bs, Cs = d["x"][bs:, :, hs].contiguous(), d["B"][bs:, :, gs:].contiguous(), C[bs:, :, gs:].contiguous()
    dts, dAs = dt[bs:, hs].contiguous(), dA[bs:, hs].contiguous()
    out_p, fin_p = _fused_chunk_state_state_passing_fwd(Bs, xs, dts, dAs, torch.bfloat16, force_general=True)
    assert_close16(out[bs:, :, hs], out_p.float().cpu(), "passed states")
    assert_close32(fin[bs:, hs], fin_p.cpu(), "final states")
    si = torch.zeros(1, l, dtype=torch.int32, device=cuda_device)      # routes to the plain kernels
    cb_p = S["bmm"](Cs, Bs, L, seq_idx=si, output_dtype=torch.float32)
    assert_close32(cb[bs:, :, gs:], cb_p.cpu(), "CB", tol=1e-5)
    y_p, _ = S["chunk_scan"](cb_p, xs, dts, dAs, Cs, out[bs:, :, hs].contiguous(), D=Dv[hs], seq_idx=si)
    assert_close16(y[bs:, :, hs], y_p.float().cpu(), "out")
