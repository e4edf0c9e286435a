"""The C interface loads without a GPU and exports exactly what include/fp6_llm_b200.h declares; argument
validation that happens before any CUDA call is checked here too."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fp6_llm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fp6b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(native_lib):
    from fp6_llm_b200 import _native
    names = declared_symbols()
    assert names == sorted(_native.C_SYMBOLS)
    for n in names:
        assert getattr(native_lib, n) is not None


def test_cxx_names_of_the_reference_are_exported(native_lib):
    from fp6_llm_b200 import _native
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", _native.LIB_PATH], capture_output=True, text=True, check=True).stdout
    for name in ("fp6_linear_kernel(", "fp_eXmY_linear_kernel(", "weight_matrix_prepacking(", "weight_matrix_prepacking_fp_eXmY(",
                 "DeQuantMatrix_FP6_To_FP16(", "dequant_matrix_fp_eXmY_to_fp16("):
        assert name in out, name


def test_version_and_error_text(native_lib):
    assert native_lib.fp6b200_version() == 2
    assert b"invalid" in native_lib.fp6b200_error_string(1).lower()


def test_host_side_validation_needs_no_gpu(native_lib):
    bad = 1   # cudaErrorInvalidValue
    assert native_lib.fp6b200_prepack_host(4, 3, None, None, 64, 64) == bad
    assert native_lib.fp6b200_prepack_host(3, 2, None, None, 64, 64) == bad
    buf = (ctypes.c_int * 1024)()
    assert native_lib.fp6b200_prepack_host(3, 2, buf, buf, 32, 64) == bad
    assert native_lib.fp6b200_dequant_host(3, 2, buf, buf, 64, 32, buf) == bad
    assert native_lib.fp6b200_splitk_reduce(None, buf, buf, 6, 2) == bad
    assert native_lib.fp6b200_workspace_bytes(4096, 8, 4096, 1) == 0
    assert native_lib.fp6b200_workspace_bytes(4096, 8, 4096, 3) == 3 * 4096 * 8 * 4


def test_python_operators_refuse_to_run_without_cuda():
    import torch
    import fp6_llm_b200 as f
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    w = torch.zeros(256, 12, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        f.weight_prepacking_cpu(w)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        f.weight_dequant_cpu(w, torch.ones(256, dtype=torch.float16))
