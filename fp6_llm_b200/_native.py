"""Builds and loads libfp6_b200.so (the CUDA kernels behind the C interface in include/fp6_llm_b200.h).

The library is compiled in-tree with nvcc for sm_100a only.  There is no fallback of any kind: if the
library is missing or fails to load, every operator raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
_CSRC = os.path.join(_PKG, "csrc")
LIB_DIR = os.path.join(_PKG, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libfp6_b200.so")
SOURCES = ("fpx_gemm.cu", "fpx_native.cu", "fpx_prepack.cu", "c_api.cu", "c_api_noalloc.cu")
HEADERS = ("fpx_internal.h", "fpx_layout.h", "ptx_sm100.cuh")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--threads", "4",
              "-Xcompiler", "-fPIC", "-shared"]

# every symbol include/fp6_llm_b200.h declares
C_SYMBOLS = (
    "fp6b200_version", "fp6b200_error_string", "fp6b200_linear", "fp6b200_linear_host_io",
    "fp6b200_workspace_bytes", "fp6b200_choose_split_k", "fp6b200_prepack", "fp6b200_prepack_host",
    "fp6b200_dequant", "fp6b200_dequant_host", "fp6b200_dequant_packed", "fp6b200_splitk_reduce",
    "fp6b200_device_status", "fp6b200_linear_static_scratch", "fp6b200_static_scratch_bytes",
    "fp6b200_linear_gather", "fp6b200_set_option", "fp6b200_get_option", "fp6b200_quantize_prepack",
    "fp6b200_linear_host_io_batch", "fp6b200_kernel_launches", "fp6b200_linear_ex",
    "fp6b200_native_supported", "fp6b200_native_preferred", "fp6b200_native_weight_bytes", "fp6b200_native_workspace_bytes",
    "fp6b200_native_repack", "fp6b200_linear_native", "fp6b200_native_kernel_launches", "fp6b200_linear_native_gather",
)


class HostCall(ctypes.Structure):
    """fp6b200_host_call of include/fp6_llm_b200.h."""
    _fields_ = [("e_bits", ctypes.c_int), ("m_bits", ctypes.c_int), ("weight_packed_dev", ctypes.c_void_p),
                ("scales_dev", ctypes.c_void_p), ("act_host", ctypes.c_void_p), ("out_host", ctypes.c_void_p),
                ("M", ctypes.c_size_t), ("N", ctypes.c_size_t), ("K", ctypes.c_size_t), ("split_k", ctypes.c_int),
                ("weight_native_dev", ctypes.c_void_p)]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libfp6_b200.so")
    return cand


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(_CSRC, f) for f in SOURCES + HEADERS]
    deps += [os.path.join(_ROOT, "include", f) for f in ("fp6_llm_b200.h", "fp6_llm_b200_cxx.cuh")]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources.  Returns its path."""
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH]
    cmd += [os.path.join(_CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library with argument types set.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()' "
            "or fp6_llm_b200.build()); there is no fallback path")
    L = ctypes.CDLL(LIB_PATH)
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    L.fp6b200_version.restype = ci
    L.fp6b200_version.argtypes = []
    L.fp6b200_error_string.restype = ctypes.c_char_p
    L.fp6b200_error_string.argtypes = [ci]
    L.fp6b200_linear.restype = ci
    L.fp6b200_linear.argtypes = [ci, ci, vp, vp, vp, vp, vp, sz, sz, sz, vp, ci]
    L.fp6b200_linear_ex.restype = ci
    L.fp6b200_linear_ex.argtypes = [ci, ci, vp, vp, vp, vp, vp, sz, sz, sz, vp, ci, vp, ci]
    L.fp6b200_native_supported.restype = ci
    L.fp6b200_native_supported.argtypes = [ci, ci, sz, sz, sz]
    L.fp6b200_native_preferred.restype = ci
    L.fp6b200_native_preferred.argtypes = [ci, ci, sz, sz, sz]
    L.fp6b200_native_weight_bytes.restype = sz
    L.fp6b200_native_weight_bytes.argtypes = [sz, sz]
    L.fp6b200_native_workspace_bytes.restype = sz
    L.fp6b200_native_workspace_bytes.argtypes = [sz, sz]
    L.fp6b200_native_repack.restype = ci
    L.fp6b200_native_repack.argtypes = [ci, ci, vp, vp, vp, sz, sz]
    L.fp6b200_linear_native.restype = ci
    L.fp6b200_linear_native.argtypes = [ci, ci, vp, vp, vp, vp, vp, sz, sz, sz, vp, vp, ci]
    L.fp6b200_linear_native_gather.restype = ci
    L.fp6b200_linear_native_gather.argtypes = [ci, ci, vp, vp, vp, vp, vp, vp, vp, ci, ci, sz, sz, sz, sz, sz, vp]
    L.fp6b200_native_kernel_launches.restype = ci
    L.fp6b200_native_kernel_launches.argtypes = [sz, sz, sz]
    L.fp6b200_linear_host_io.restype = ci
    L.fp6b200_linear_host_io.argtypes = [ci, ci, vp, vp, vp, vp, sz, sz, sz, ci]
    L.fp6b200_linear_host_io_batch.restype = ci
    L.fp6b200_linear_host_io_batch.argtypes = [ctypes.POINTER(HostCall), ci]
    L.fp6b200_kernel_launches.restype = ci
    L.fp6b200_kernel_launches.argtypes = [sz, sz, sz, ci]
    L.fp6b200_workspace_bytes.restype = sz
    L.fp6b200_workspace_bytes.argtypes = [sz, sz, sz, ci]
    L.fp6b200_choose_split_k.restype = ci
    L.fp6b200_choose_split_k.argtypes = [sz, sz, sz, ci]
    L.fp6b200_prepack.restype = ci
    L.fp6b200_prepack.argtypes = [ci, ci, vp, vp, vp, sz, sz]
    L.fp6b200_prepack_host.restype = ci
    L.fp6b200_prepack_host.argtypes = [ci, ci, vp, vp, sz, sz]
    L.fp6b200_dequant.restype = ci
    L.fp6b200_dequant.argtypes = [ci, ci, vp, vp, vp, vp, sz, sz]
    L.fp6b200_dequant_host.restype = ci
    L.fp6b200_dequant_host.argtypes = [ci, ci, vp, vp, sz, sz, vp]
    L.fp6b200_dequant_packed.restype = ci
    L.fp6b200_dequant_packed.argtypes = [ci, ci, vp, vp, vp, vp, sz, sz]
    L.fp6b200_splitk_reduce.restype = ci
    L.fp6b200_splitk_reduce.argtypes = [vp, vp, vp, sz, ci]
    L.fp6b200_linear_static_scratch.restype = ci
    L.fp6b200_linear_static_scratch.argtypes = [ci, ci, vp, vp, vp, vp, vp, sz, sz, sz]
    L.fp6b200_static_scratch_bytes.restype = sz
    L.fp6b200_static_scratch_bytes.argtypes = []
    L.fp6b200_linear_gather.restype = ci
    L.fp6b200_linear_gather.argtypes = [ci, ci, vp, vp, vp, vp, vp, vp, vp, ci, ci, sz, sz, sz, sz, sz, vp, ci]
    L.fp6b200_set_option.restype = ci
    L.fp6b200_set_option.argtypes = [ci, ci]
    L.fp6b200_get_option.restype = ci
    L.fp6b200_get_option.argtypes = [ci]
    L.fp6b200_quantize_prepack.restype = ci
    L.fp6b200_quantize_prepack.argtypes = [ci, ci, vp, vp, vp, vp, sz, sz]
    L.fp6b200_device_status.restype = ci
    L.fp6b200_device_status.argtypes = [ctypes.POINTER(ci)]
    _lib = L
    return L


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().fp6b200_error_string(code)
        raise RuntimeError(f"{what} failed: CUDA error {code} ({msg.decode() if msg else '?'})")
