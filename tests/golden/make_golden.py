"""Generate the golden fixtures in this directory from the REFERENCE's own kernels.

Two modes:

  python tests/golden/make_golden.py --reference /path/to/mamba-fused-minimal --mode interp
      Runs the reference's Triton kernels on the CPU under TRITON_INTERPRET=1 (no GPU
      needed).  Only fp32 inputs: the interpreter does not execute bf16 arithmetic
      faithfully.  Writes interp_*.npz.

  python tests/golden/make_golden.py --reference /path/to/mamba-fused-minimal --mode gpu
      Runs the reference's compiled Triton kernels (the five original, unfused kernels,
      which contain no spin-waits) on the current CUDA device with bf16 / fp16 inputs.
      Writes gpu_*.npz.

The reference tree is only read (imported); nothing is copied from it.  Harness-side
adjustments in interpreter mode, none touching reference files: `torch.cuda.device` becomes
a null context (the wrappers enter it with a None index on a CUDA-less build), every
autotuner keeps one configuration (benchmarking configurations needs a GPU), and for the
global-barrier kernel the device is reported as having one multiprocessor so that its
single program passes its own barrier.

Inputs are stored in the fixture next to the outputs, so the tests need neither the
reference nor this script.
"""
import argparse
import contextlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def _np(t):
    import torch
    if t is None or isinstance(t, np.ndarray):
        return t
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        # store 16-bit floats as their bit patterns; the dtype name is stored beside them
        return t.view(torch.int16).numpy()
    return t.numpy()


def save(path, dtype_name, **tensors):
    arrays = {k: _np(v) for k, v in tensors.items() if v is not None}
    arrays["_dtype"] = np.array(dtype_name)
    np.savez_compressed(path, **arrays)
    print("wrote", path, {k: getattr(v, "shape", None) for k, v in arrays.items()})


CASES = {
    # name: (batch, seqlen, nheads, headdim, ngroups, dstate, chunk_size, options)
    "cfg0": (1, 512, 4, 32, 1, 16, 64, dict(softplus=True, bias=True, D="h")),
    "ragged": (2, 200, 4, 32, 2, 16, 64, dict(softplus=True, bias=True, D="hp", z=True,
                                                init=True)),
    "limits": (1, 160, 2, 16, 1, 32, 32, dict(softplus=False, bias=True, D=None,
                                               dt_limit=(0.6, 0.9), refstyle=True)),
    "seqidx": (2, 192, 2, 16, 1, 16, 64, dict(softplus=True, bias=False, D="h",
                                               seq_idx=True)),
}
GPU_CASES = {
    "bf16_small": (2, 384, 4, 64, 2, 128, 128, dict(softplus=True, bias=True, D="h", init=True)),
    "bf16_ragged": (1, 300, 3, 64, 1, 64, 64, dict(softplus=True, bias=True, D="hp", z=True)),
    "fp16_small": (1, 256, 2, 32, 1, 32, 64, dict(softplus=True, bias=True, D="h")),
    # packed sequences + gate + ragged last chunk at a shape every tcgen05 kernel takes
    "bf16_packed": (1, 400, 2, 64, 1, 128, 128, dict(softplus=True, bias=True, D="hp", z=True, seq_idx=True)),
}


def build_inputs(case, dtype, device):
    import torch
    from oracle import ssd_oracle as O
    b, l, h, p, g, n, L, opt = case
    if opt.get("refstyle"):
        d = O.make_inputs_reference_style(b, l, h, p, g, n, dtype=dtype, seed=42)
    else:
        d = O.make_inputs(b, l, h, p, g, n, dtype=dtype, seed=0)
    gen = torch.Generator().manual_seed(1234)
    if not opt.get("bias"):
        d["dt_bias"] = None
    if opt.get("D") == "hp":
        d["D"] = torch.randn(h, p, generator=gen)
    elif opt.get("D") is None:
        d["D"] = None
    d["z"] = torch.randn(b, l, h, p, generator=gen).to(dtype) if opt.get("z") else None
    d["init"] = torch.randn(b, h, p, n, generator=gen) if opt.get("init") else None
    if opt.get("seq_idx"):
        # three packed sequences with boundaries inside and on chunk edges
        si = torch.zeros(b, l, dtype=torch.int32)
        si[:, 50:] = 1
        si[:, 128:] = 2
        d["seq_idx"] = si
    else:
        d["seq_idx"] = None
    return {k: (v.to(device) if v is not None else None) for k, v in d.items()}


def run_reference(mods, d, L, opt):
    """The unfused pipeline of the reference's main.py:60-74, piece by piece so that each
    intermediate is captured; initial_states / seq_idx forwarded where its functions take
    them."""
    import torch
    cs, sp, bm, sc = mods
    x, dt, A, B, C = d["x"], d["dt"], d["A"], d["B"], d["C"]
    dt_limit = opt.get("dt_limit", (0.0, float("inf")))
    dA_cumsum, dt_out = cs._chunk_cumsum_fwd(dt, A, L, dt_bias=d["dt_bias"],
                                             dt_softplus=opt.get("softplus", False),
                                             dt_limit=dt_limit)
    states = cs._chunk_state_fwd(B, x, dt_out, dA_cumsum, seq_idx=d["seq_idx"],
                                 states_in_fp32=True)
    bsz, nchunks, h, p, n = states.shape
    init = d["init"]
    passed, final = sp._state_passing_fwd(
        states.reshape(bsz, nchunks, h, p * n), dA_cumsum[:, :, :, -1],
        initial_states=None if init is None else init.reshape(bsz, h, p * n),
        seq_idx=d["seq_idx"], chunk_size=L, out_dtype=C.dtype)
    passed = passed.view(bsz, nchunks, h, p, n)
    final = final.view(bsz, h, p, n)
    CB = bm._bmm_chunk_fwd(C, B, L, seq_idx=d["seq_idx"], output_dtype=torch.float32)
    out, out_x = sc._chunk_scan_fwd(CB, x, dt_out, dA_cumsum, C, passed, D=d["D"], z=d["z"],
                                    seq_idx=d["seq_idx"])
    return dict(o_dA_cumsum=dA_cumsum, o_dt=dt_out, o_states=states, o_passed=passed,
                o_final=final, o_CB=CB, o_out=out, o_out_x=out_x)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--mode", choices=["interp", "gpu"], required=True)
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--only", default=None, help="write this one case only")
    args = ap.parse_args()
    if args.mode == "interp":
        os.environ["TRITON_INTERPRET"] = "1"
    import torch
    sys.path.insert(0, args.reference)
    if args.mode == "interp":
        torch.cuda.device = lambda *a, **k: contextlib.nullcontext()
    import kernels.ssd_chunk_state as cs
    import kernels.ssd_state_passing as sp
    import kernels.ssd_bmm as bm
    import kernels.ssd_chunk_scan as sc
    mods = (cs, sp, bm, sc)
    if args.mode == "interp":
        import kernels.fused_globalbar as gb
        for mod in mods + (gb,):
            for name in dir(mod):
                obj = getattr(mod, name)
                if isinstance(getattr(obj, "configs", None), list):
                    obj.configs = obj.configs[-1:]
        for name, case in CASES.items():
            if args.only not in (None, name):
                continue
            opt = case[-1]
            d = build_inputs(case, torch.float32, "cpu")
            res = run_reference(mods, d, case[6], opt)
            if name == "cfg0":
                # the fused global-barrier entry point with a single program
                class _P:
                    multi_processor_count = 1
                real_props, real_zeros = torch.cuda.get_device_properties, torch.zeros
                torch.cuda.get_device_properties = lambda *a, **k: _P()
                torch.zeros = lambda *a, **k: real_zeros(
                    *a, **{kk: ("cpu" if kk == "device" else vv) for kk, vv in k.items()})
                try:
                    fo, ff = gb._fused_chunk_state_state_passing_fwd_globalbar(
                        d["B"], d["x"], res["o_dt"], res["o_dA_cumsum"], d["C"].dtype,
                        initial_states=None, seq_idx=None, states_in_fp32=True)
                finally:
                    torch.cuda.get_device_properties, torch.zeros = real_props, real_zeros
                res["o_fused_out"], res["o_fused_final"] = fo, ff
            meta = np.array(list(case[:7]), dtype=np.int64)
            save(os.path.join(args.out, f"interp_{name}.npz"), "float32", meta=meta,
                 dt_limit=torch.tensor(opt.get("dt_limit", (0.0, float("inf")))),
                 softplus=torch.tensor(int(opt.get("softplus", False))), **d, **res)
    else:
        for name, case in GPU_CASES.items():
            if args.only not in (None, name):
                continue
            opt = case[-1]
            dtype = torch.float16 if name.startswith("fp16") else torch.bfloat16
            d = build_inputs(case, dtype, "cuda")
            res = run_reference(mods, d, case[6], opt)
            torch.cuda.synchronize()
            meta = np.array(list(case[:7]), dtype=np.int64)
            save(os.path.join(args.out, f"gpu_{name}.npz"), str(dtype).split(".")[-1],
                 meta=meta, dt_limit=torch.tensor(opt.get("dt_limit", (0.0, float("inf")))),
                 softplus=torch.tensor(int(opt.get("softplus", False))), **d, **res)


if __name__ == "__main__":
    main()
