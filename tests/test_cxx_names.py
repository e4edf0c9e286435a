"""The reference's C++ interface (fp6_llm/csrc/fp6_linear.cuh:8-43), used through its mangled names: a small program
includes include/fp6_llm_b200_cxx.cuh, links libfp6_b200.so and calls fp6_linear_kernel, fp_eXmY_linear_kernel,
weight_matrix_prepacking (in place, as the reference's tests/cpp do) and DeQuantMatrix_FP6_To_FP16.  Compiling and
linking is checked everywhere (nvcc cross-compiles without a GPU); running it and comparing with the oracle needs a GPU."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def program(tmp_path_factory, native_lib):
    from fp6_llm_b200 import _native
    exe = str(tmp_path_factory.mktemp("cxx") / "reference_names")
    cmd = [_native._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cxx", "reference_names.cu"), "-o", exe,
           "-L", _native.LIB_DIR, "-lfp6_b200", "-Xlinker", "-rpath", "-Xlinker", _native.LIB_DIR]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stdout + done.stderr
    return exe


def test_program_links_against_the_reference_names(program):
    out = subprocess.run(["nm", "-u", "-C", program], capture_output=True, text=True, check=True).stdout
    for name in ("fp6_linear_kernel(", "fp_eXmY_linear_kernel(", "weight_matrix_prepacking(", "DeQuantMatrix_FP6_To_FP16("):
        assert name in out, name


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,split_k", [(512, 12, 1024, 1), (256, 70, 2048, 3)])
def test_program_results_match_the_oracle(program, oracle_mod, tmp_path, M, N, K, split_k):
    from helpers import random_unpacked
    rng = np.random.default_rng(M + N)
    w = random_unpacked(rng, M, K, 3, 2)
    s = rng.uniform(0.01, 0.1, M).astype(np.float16)
    x = rng.standard_normal((N, K)).astype(np.float16)
    w.tofile(tmp_path / "weights.bin")
    s.tofile(tmp_path / "scales.bin")
    x.tofile(tmp_path / "act.bin")
    done = subprocess.run([program, str(tmp_path), str(M), str(N), str(K), str(split_k)], capture_output=True, text=True)
    assert done.returncode == 0 and "ok" in done.stdout, done.stdout + done.stderr
    packed = np.fromfile(tmp_path / "packed.bin", dtype=np.int32).reshape(w.shape)
    assert np.array_equal(packed, oracle_mod.prepack(w, 3, 2))                       # in place, bit-exact
    deq = np.fromfile(tmp_path / "dequant.bin", dtype=np.float16).reshape(M, K)
    assert np.array_equal(deq.view(np.uint16), oracle_mod.dequant(w, s, 3, 2).view(np.uint16))
    truth = oracle_mod.linear(x, w, s, 3, 2)
    for name in ("out.bin", "out_exmy.bin"):
        y = np.fromfile(tmp_path / name, dtype=np.float16).reshape(N, M).astype(np.float32)
        res = oracle_mod.check_tolerance(y, truth)
        assert res["rel_fro"] <= 2e-3 and res["max_row_rel"] <= 1e-2, res
