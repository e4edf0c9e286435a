"""TEST INFRASTRUCTURE ONLY: ctypes/numpy front end of the CPU oracle.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package.  The shipped library (``fp6_llm_b200``) never does.

``oracle.*``      -> the plain-C restatement in ``fpx_oracle.c``
``oracle.ref_*``  -> the reference's own CPU functions, when ``oracle/_ref`` was
                     built from the reference sources (see ``oracle/Makefile``)

Reference call sites this mirrors: ``weight_matrix_prepacking_fp_eXmY``
(fp6_llm/csrc/utils/weight_prepacking.h:204-211), ``dequant_matrix_fp_eXmY_to_fp16``
(fp6_llm/csrc/utils/weight_dequant.h:54-61) and the tests' ground truth
"dequantise, then fp16/fp32 matmul" (tests/python/kernel_test_fp6.py:48-58).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "_build", "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libfp6_ref.so")
_REF_GPU_SO = os.path.join(_HERE, "_ref", "libfp6_ref_gpu.so")


def _find_reference() -> str | None:
    """A checkout of the reference project: $FP6_LLM_REFERENCE, else a `reference` folder beside this repository."""
    cand = [os.environ.get("FP6_LLM_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cand:
        if c and os.path.isdir(os.path.join(c, "fp6_llm", "csrc")):
            return c
    return None


def build(reference_root: str | None = None) -> None:
    """Compile the C restatement and, when a checkout of the reference is found, oracle/_ref from its sources."""
    args = ["make", "-s", "-C", _HERE, "all"]
    reference_root = reference_root or _find_reference()
    if reference_root:
        args.append(f"REFERENCE_ROOT={reference_root}")
        args.append("refgpu")      # the reference's GPU kernel recompiled for sm_100a: the benchmark's same-box comparison
    subprocess.run(args, check=True)


def _load(path):
    return ctypes.CDLL(path)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_ORACLE_SO):
            build()
        _lib = _load(_ORACLE_SO)
        _lib.oracle_prepack.restype = ctypes.c_int
        _lib.oracle_prepack.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_size_t, ctypes.c_size_t]
        _lib.oracle_dequant.restype = ctypes.c_int
        _lib.oracle_dequant.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p]
        _lib.oracle_splitk_reduce.restype = None
        _lib.oracle_splitk_reduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        _lib.oracle_float_to_half.restype = ctypes.c_uint16
        _lib.oracle_float_to_half.argtypes = [ctypes.c_float]
        _lib.oracle_half_to_float.restype = ctypes.c_float
        _lib.oracle_half_to_float.argtypes = [ctypes.c_uint16]
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF_SO)


_ref_gpu = None


def have_ref_gpu() -> bool:
    return os.path.exists(_REF_GPU_SO)


def ref_gpu():
    """The reference's own GPU launcher (fp_eXmY_linear_kernel, fp6_llm/csrc/fp6_linear.cuh:20-32) recompiled for sm_100a:
    ref_gpu().ref_gpu_linear(e, m, stream, weight, scales, act, out, M, N, K, workspace, split_k) on device pointers."""
    global _ref_gpu
    if _ref_gpu is None:
        _ref_gpu = _load(_REF_GPU_SO)
        vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        _ref_gpu.ref_gpu_linear.restype = ci
        _ref_gpu.ref_gpu_linear.argtypes = [ci, ci, vp, vp, vp, vp, vp, sz, sz, sz, vp, ci]
    return _ref_gpu


def ref():
    global _ref
    if _ref is None:
        _ref = _load(_REF_SO)
        _ref.ref_prepack.restype = ctypes.c_int
        _ref.ref_prepack.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_size_t, ctypes.c_size_t]
        _ref.ref_dequant.restype = ctypes.c_int
        _ref.ref_dequant.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p]
    return _ref


def _shape(w: np.ndarray, e: int, m: int):
    bw = 1 + e + m
    assert w.dtype == np.int32 and w.ndim == 2 and w.flags.c_contiguous
    rows, words = w.shape
    assert (words * 32) % bw == 0
    return rows, words * 32 // bw


def _prepack_with(fn, w, e, m):
    rows, cols = _shape(w, e, m)
    out = np.empty_like(w)
    rc = fn(e, m, out.ctypes.data, w.ctypes.data, rows, cols)
    if rc != 0:
        raise ValueError(f"prepack rejected e{e}m{m} {rows}x{cols}")
    return out


def _dequant_with(fn, w, scale, e, m):
    rows, cols = _shape(w, e, m)
    scale = np.ascontiguousarray(scale, dtype=np.float16)
    assert scale.shape == (rows,)
    out = np.empty((rows, cols), dtype=np.float16)
    # one spare byte: the reference reads Bytes[ByteOffset+1] unconditionally (common.h:10)
    buf = np.zeros(w.nbytes + 8, dtype=np.uint8)
    buf[: w.nbytes] = w.view(np.uint8).reshape(-1)
    rc = fn(e, m, out.ctypes.data, buf.ctypes.data, rows, cols, scale.ctypes.data)
    if rc != 0:
        raise ValueError(f"dequant rejected e{e}m{m} {rows}x{cols}")
    return out


def prepack(w: np.ndarray, e: int = 3, m: int = 2) -> np.ndarray:
    """Unpacked int32 [OC, IC*bw/32] -> prepacked int32 of the same shape (C restatement)."""
    return _prepack_with(lib().oracle_prepack, w, e, m)


def dequant(w: np.ndarray, scale: np.ndarray, e: int = 3, m: int = 2) -> np.ndarray:
    """Unpacked int32 [OC, IC*bw/32] + fp16 scale [OC] -> fp16 [OC, IC] (C restatement)."""
    return _dequant_with(lib().oracle_dequant, w, scale, e, m)


def ref_prepack(w: np.ndarray, e: int = 3, m: int = 2) -> np.ndarray:
    return _prepack_with(ref().ref_prepack, w, e, m)


def ref_dequant(w: np.ndarray, scale: np.ndarray, e: int = 3, m: int = 2) -> np.ndarray:
    return _dequant_with(ref().ref_dequant, w, scale, e, m)


def linear(x: np.ndarray, w_unpacked: np.ndarray, scale: np.ndarray, e: int = 3, m: int = 2,
           use_ref: bool = False) -> np.ndarray:
    """Ground truth of the linear layer: dequantise to fp16, then an fp32 matmul.  Returns fp32 [BS, OC]."""
    w16 = (ref_dequant if use_ref else dequant)(w_unpacked, scale, e, m)
    return x.astype(np.float32) @ w16.astype(np.float32).T


def splitk_reduce(partials: np.ndarray) -> np.ndarray:
    """fp32 [split, ...] -> fp16 [...]: ascending fp32 sum, one round-to-nearest (kernel_reduction.cuh:28-47)."""
    partials = np.ascontiguousarray(partials, dtype=np.float32)
    out = np.empty(partials.shape[1:], dtype=np.float16)
    lib().oracle_splitk_reduce(out.ctypes.data, partials.ctypes.data, out.size, partials.shape[0])
    return out


def check_tolerance(y: np.ndarray, y_ref: np.ndarray) -> dict:
    """The two GEMM acceptance numbers: relative Frobenius error (<= 2e-3) and the worst
    max-abs error of a row relative to that row's largest reference magnitude (<= 1e-2)."""
    y = y.astype(np.float64)
    y_ref = y_ref.astype(np.float64)
    fro = float(np.linalg.norm(y - y_ref) / max(np.linalg.norm(y_ref), 1e-30))
    row_inf = np.maximum(np.abs(y_ref).max(axis=1), 1e-30)
    row_err = np.abs(y - y_ref).max(axis=1) / row_inf
    return {"rel_fro": fro, "max_row_rel": float(row_err.max()),
            "ok": bool(fro <= 2e-3 and row_err.max() <= 1e-2)}
