"""Loads the prebuilt native modules.  There is no fallback: if the C-ABI library or the
PyTorch front end is missing, importing this module raises with the build command."""
import ctypes
import importlib.util
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libssd_b200.so")
EXT_PATH = os.path.join(PKG, "_C.so")

_BUILD_HINT = "run `python -m mamba_fused_minimal_b200.build` (needs nvcc and g++)"


def load_abi():
    """The C-ABI library as a ctypes handle (symbols of include/ssd_b200.h)."""
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: {_BUILD_HINT}")
    return ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)


def _load_ext():
    if not os.path.exists(LIB_PATH) or not os.path.exists(EXT_PATH):
        raise ImportError(f"native modules are missing under {PKG}: {_BUILD_HINT}")
    import torch  # noqa: F401  (the extension links against the torch libraries)
    spec = importlib.util.spec_from_file_location("mamba_fused_minimal_b200._C", EXT_PATH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


C = _load_ext()
