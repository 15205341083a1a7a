"""The ctypes binding printed in INTEGRATION.md, executed as printed.

INTEGRATION.md shows the stub a maintainer of the reference would put in place of the body of
`_fused_chunk_state_state_passing_fwd_concurrent` (kernels/fused_concurrent.py:255-331 there) to
call the C ABI without the PyTorch C++ extension.  This test extracts that code block from the
file, executes it (the only edit: the bare library name is replaced by the library's path in
this tree, since the test does not install it on the loader's search path) and compares the
function it defines with the extension's on the same inputs.  A drift between the struct
layouts in the document and include/ssd_b200.h shows up here."""
import os
import re

import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _stub_source():
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    stubs = [b for b in blocks if "ctypes.CDLL" in b and "class FusedParams" in b]
    assert len(stubs) == 1, "INTEGRATION.md should hold exactly one ctypes stub"
    return stubs[0]


def test_the_documented_ctypes_stub_runs_and_agrees(cuda_device):
    from mamba_fused_minimal_b200._ext import LIB_PATH
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as ext_fn
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    src = _stub_source()
    assert 'ctypes.CDLL("libssd_b200.so")' in src
    src = src.replace('ctypes.CDLL("libssd_b200.so")', f"ctypes.CDLL({LIB_PATH!r})")
    ns = {}
    exec(compile(src, "INTEGRATION.md:ctypes-stub", "exec"), ns)
    stub_fn = ns["_fused_chunk_state_state_passing_fwd_concurrent"]
    for shape, dtype, with_init in [((2, 2048, 8, 64, 1, 128, 256), torch.bfloat16, True),
                                    ((1, 8192, 2, 64, 1, 128, 64), torch.bfloat16, False),     # carries between CTAs
                                    ((2, 320, 4, 32, 2, 16, 64), torch.float32, True)]:        # plain kernels
        b, l, h, p, g, n, L = shape
        inp = {k: v.to(cuda_device) for k, v in O.make_inputs(b, l, h, p, g, n, dtype=dtype, seed=61).items()}
        dA, dt = _chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
        init = torch.randn(b, h, p, n, device=cuda_device) if with_init else None
        for _ in range(2):                       # the stub's workspace is zeroed once and then reused
            out_s, fin_s = stub_fn(inp["B"], inp["x"], dt, dA, dtype, initial_states=init)
            out_e, fin_e = ext_fn(inp["B"], inp["x"], dt, dA, dtype, initial_states=init)
            torch.cuda.synchronize()
            assert torch.equal(out_s, out_e) and torch.equal(fin_s, fin_e)
