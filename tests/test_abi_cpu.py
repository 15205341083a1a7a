"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares,
rejects bad arguments without touching a device, and the Python layer fails loudly when
asked to run without CUDA."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ssd_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"SSD_API\s+[\w\s\*]+?\b(ssd_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for s in ["ssd_chunk_cumsum_fwd", "ssd_chunk_state_fwd", "ssd_state_passing_fwd", "ssd_fused_state_fwd",
              "ssd_fused_state_workspace_bytes", "ssd_bmm_chunk_fwd", "ssd_chunk_scan_fwd", "ssd_check_status",
              "ssd_last_error", "ssd_abi_version", "ssd_state_path_fwd", "ssd_state_path_workspace_bytes",
              "ssd_chunk_scan_fused_fwd", "ssd_combined_fwd", "ssd_seqpar_fixup", "ssd_fused_state_fwd_static",
              "ssd_debug_set_wait_limit_cycles", "ssd_debug_set_flags"]:
        assert s in syms


def test_library_exports_every_declared_symbol():
    from mamba_fused_minimal_b200._ext import load_abi
    lib = load_abi()
    for s in declared_symbols():
        assert hasattr(lib, s), s
    assert lib.ssd_abi_version() == 1


def test_null_params_are_rejected_with_a_message():
    from mamba_fused_minimal_b200._ext import load_abi
    lib = load_abi()
    lib.ssd_last_error.restype = ctypes.c_char_p
    for fn in ["ssd_chunk_cumsum_fwd", "ssd_chunk_state_fwd", "ssd_state_passing_fwd", "ssd_fused_state_fwd",
               "ssd_bmm_chunk_fwd", "ssd_chunk_scan_fwd", "ssd_state_path_fwd", "ssd_chunk_scan_fused_fwd",
               "ssd_combined_fwd", "ssd_seqpar_fixup", "ssd_fused_state_fwd_static"]:
        rc = getattr(lib, fn)(None, None)
        assert rc == 1, fn                       # SSD_ERR_BAD_ARGUMENT
        assert b"NULL" in lib.ssd_last_error()


def test_python_layer_refuses_cpu_tensors():
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    with pytest.raises(RuntimeError, match="no CPU path"):
        _chunk_cumsum_fwd(torch.zeros(1, 8, 2), torch.zeros(2), 4)


def test_shape_assertions_match_the_reference_convention():
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd, _chunk_state_fwd
    with pytest.raises(AssertionError):
        _chunk_cumsum_fwd(torch.zeros(1, 8, 2), torch.zeros(3), 4)
    with pytest.raises(AssertionError):
        _chunk_state_fwd(torch.zeros(1, 8, 1, 4), torch.zeros(1, 8, 2, 4), torch.zeros(1, 2, 2, 4),
                         torch.zeros(1, 2, 2, 5))
