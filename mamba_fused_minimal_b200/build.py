"""In-tree build of the native parts.

  libssd_b200.so   the C-ABI library: hand-written CUDA for sm_100a (nvcc, static cudart)
  _C.so            the PyTorch C++ front end (g++ against the torch headers), linked to
                   libssd_b200.so through an $ORIGIN rpath
  tma_copy_probe   a stand-alone diagnostic binary (how fast the state kernel's tiles move with TMA alone)

Both land next to this file so that they travel with the source tree.  Nothing is built at
import time on a machine without the toolchain: `mamba_fused_minimal_b200._ext` loads the
prebuilt files and raises if they are missing.

    python -m mamba_fused_minimal_b200.build [--force] [--verbose]
"""
import argparse
import hashlib
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")

CUDA_SOURCES = ["ssd_abi.cu", "ssd_general.cu", "ssd_fused_sm100.cu", "ssd_gemm_sm100.cu", "ssd_static_scratch.cu"]
CUDA_HEADERS = ["ssd_common.cuh", "ssd_carry.cuh", "ssd_launch.h", "sm100_ptx.cuh", os.path.join(INCLUDE, "ssd_b200.h")]
LIB = os.path.join(PKG, "libssd_b200.so")
EXT = os.path.join(PKG, "_C.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
PROBE = os.path.join(PKG, "tma_copy_probe")


def _nvcc():
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return os.path.join(home, "bin", "nvcc")


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target, stamp_value):
    stamp = target + ".stamp"
    if not os.path.exists(target) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != stamp_value


def _write_stamp(target, stamp_value):
    with open(target + ".stamp", "w") as f:
        f.write(stamp_value)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    if verbose:
        sys.stdout.write(res.stdout + res.stderr)


def build_lib(force=False, verbose=False):
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in CUDA_HEADERS]
    flags = NVCC_FLAGS + os.environ.get("SSD_EXTRA_NVCC_FLAGS", "").split()
    stamp = _digest(srcs + hdrs, " ".join(flags))
    if not force and not _stale(LIB, stamp):
        return LIB
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(PKG, "build", os.path.basename(s) + ".o")
        os.makedirs(os.path.dirname(o), exist_ok=True)
        cmd = [_nvcc()] + flags + ["-I" + INCLUDE, "-I" + CSRC, "-c", s, "-o", o]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(o)
    for cmd, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError("build step failed: " + " ".join(cmd))
        if verbose:
            sys.stdout.write(out)
    _run([_nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    _write_stamp(LIB, stamp)
    return LIB


def build_ext(force=False, verbose=False):
    import torch
    from torch.utils import cpp_extension as ce
    src = os.path.join(CSRC, "torch_ext.cpp")
    stamp = _digest([src, os.path.join(INCLUDE, "ssd_b200.h")], torch.__version__)
    if not force and not _stale(EXT, stamp):
        return EXT
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include"), INCLUDE]
    libdirs = ce.library_paths()
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), src, "-o", EXT]
    cmd += ["-I" + p for p in inc]
    cmd += ["-L" + p for p in libdirs] + ["-L" + PKG]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-l:libssd_b200.so"]
    cmd += ["-Wl,-rpath,$ORIGIN"] + ["-Wl,-rpath," + p for p in libdirs]
    _run(cmd, verbose)
    _write_stamp(EXT, stamp)
    return EXT


def build_probe(force=False, verbose=False):
    """The stand-alone copy-engine probe (csrc/tma_copy_probe.cu): what the state kernel's tiles cost to
    move with TMA alone.  A diagnostic for the roofline discussion; nothing in the library uses it."""
    src = os.path.join(CSRC, "tma_copy_probe.cu")
    stamp = _digest([src])
    if not force and not _stale(PROBE, stamp):
        return PROBE
    _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", PROBE, src, "-lcuda"], verbose)
    _write_stamp(PROBE, stamp)
    return PROBE


def build_all(force=False, verbose=False):
    build_lib(force, verbose)
    build_ext(force, verbose)
    build_probe(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    build_all(a.force, a.verbose)
    print("built", LIB, EXT)
