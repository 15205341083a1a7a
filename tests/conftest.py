import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name):
    """Load a fixture written by tests/golden/make_golden.py into torch tensors."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    dtype_name = str(z["_dtype"])
    dtype = getattr(torch, dtype_name)
    out = {}
    for k in z.files:
        if k == "_dtype":
            continue
        a = z[k]
        t = torch.from_numpy(a.copy()) if a.ndim else torch.tensor(a.item())
        if a.dtype == np.int16:      # 16-bit floats are stored as bit patterns
            t = t.view(dtype)
        out[k] = t
    out["_dtype"] = dtype
    return out


def golden_names(prefix):
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.startswith(prefix) and f.endswith(".npz"))


def rel_err(a, b):
    """max|a-b| / max|b|: the error measure the state tolerance is stated in."""
    a = a.float()
    b = b.float()
    denom = b.abs().max().item()
    return (a - b).abs().max().item() / max(denom, 1e-30)


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(params=["layout_chosen", "layout_ranges_per_sm"])
def both_layouts(request, cuda_device):
    """Runs a test twice: with the layout the fused state kernel chooses for the problem (small
    test problems run one CTA per head over whole strips) and with the test hook
    SSD_DEBUG_CUT_STRIPS, which forces the layout of large problems (one range of (strip, chunk)
    items per SM, states carried between CTAs through carry slots and flags) on the same inputs."""
    from mamba_fused_minimal_b200._ext import C
    C.debug_set_flags(2 if request.param == "layout_ranges_per_sm" else 0)
    try:
        yield request.param
    finally:
        C.debug_set_flags(0)
