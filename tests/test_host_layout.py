"""The integer layout/unpack code shared with the CUDA kernels (fp6_llm_b200/csrc/fpx_layout.h), compiled for the
host and compared with the oracle: the prepack gather, the registers every lane of the GEMM produces and where the
tensor-memory store puts them, and the split-K ranges."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from helpers import ALL_FORMATS, random_unpacked

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    so = str(tmp_path_factory.mktemp("harness") / "liblayout_harness.so")
    subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-o", so,
                    os.path.join(HERE, "host", "layout_harness.cpp")], check=True)
    return ctypes.CDLL(so)


@pytest.mark.parametrize("e,m", ALL_FORMATS)
@pytest.mark.parametrize("rows,cols", [(128, 64), (256, 192), (384, 320)])
def test_prepack_gather_matches_oracle(harness, oracle_mod, e, m, rows, cols):
    rng = np.random.default_rng(rows + cols + e)
    w = random_unpacked(rng, rows, cols, e, m)
    out = np.zeros_like(w)
    assert harness.harness_prepack(e, m, ctypes.c_void_p(out.ctypes.data), ctypes.c_void_p(w.ctypes.data), rows, cols) == 0
    assert np.array_equal(out, oracle_mod.prepack(w, e, m))


@pytest.mark.parametrize("e,m", ALL_FORMATS)
@pytest.mark.parametrize("rows,cols", [(128, 64), (256, 256)])
def test_gemm_unpack_registers(harness, oracle_mod, e, m, rows, cols):
    rng = np.random.default_rng(rows * 3 + cols + e)
    w = random_unpacked(rng, rows, cols, e, m)
    packed = oracle_mod.prepack(w, e, m)
    bits = np.zeros((rows, cols), np.uint16)
    assert harness.harness_unpack(e, m, ctypes.c_void_p(bits.ctypes.data), ctypes.c_void_p(packed.ctypes.data), rows, cols) == 0
    expect = oracle_mod.dequant(w, np.ones(rows, np.float16), e, m).astype(np.float32)
    bias = np.array([harness.harness_bias_bits(e)], np.uint16).view(np.float16).astype(np.float32)[0]
    assert bias == 2.0 ** (16 - 2 ** (e - 1))
    got = bits.view(np.float16).astype(np.float32) * bias
    assert np.array_equal(got, expect) and np.array_equal(np.signbit(got), np.signbit(expect))


def test_split_ranges_cover_k(harness):
    harness.harness_split_range.argtypes = [ctypes.c_uint32] * 3 + [ctypes.POINTER(ctypes.c_uint32)] * 2
    for kb in (1, 2, 7, 64, 172, 448):
        for splits in (1, 2, 3, 7, kb, kb + 3):
            nxt = 0
            for z in range(splits):
                b, c = ctypes.c_uint32(), ctypes.c_uint32()
                harness.harness_split_range(kb, splits, z, ctypes.byref(b), ctypes.byref(c))
                # reference: avg (+1 for the first `extra` splits), fp6_llm/csrc/include/kernel_matmul.cuh:60-70
                assert c.value == kb // splits + (1 if z < kb % splits else 0)
                assert b.value == nxt
                nxt += c.value
            assert nxt == kb


def test_work_plans_cover_every_unit_once(harness):
    """Classic split-K and the wave + stream-K plan: every (tile, K block) is covered exactly once, and the slots
    the fix-up kernel sums are exactly the partial segments the GEMM CTAs write."""
    import itertools
    n = 0
    for mode in (0, 1):
        for mt, nt, kb, grid in itertools.product((1, 2, 3, 32, 86, 96, 172, 448), (1, 2, 9), (1, 2, 7, 64, 172), (1, 2, 3, 147, 148)):
            for sk in ((1, 2, 3, 5, kb) if mode == 0 else (1,)):
                if sk > kb:
                    continue
                assert harness.harness_check_plan(mode, mt, nt, kb, sk, grid) == 0, (mode, mt, nt, kb, sk, grid)
                n += 1
    assert n > 1000


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_quantiser_matches_the_tensor_quantiser(harness, e, m):
    """The scalar round-to-nearest routine of the fused quantise + pack kernel against formats.quantize_rtn, on random
    quotients, on every magnitude, on every exact tie between neighbours, beyond the largest magnitude and on signed
    zeros."""
    import torch
    from fp6_llm_b200.formats import magnitudes, quantize_rtn
    mag = magnitudes(e, m)
    mids = (mag[:-1] + mag[1:]) * 0.5
    gen = torch.Generator().manual_seed(11 + e)
    q = torch.cat([torch.randn(20000, generator=gen) * float(mag[-1]) * 0.5, mag, -mag, mids, -mids,
                   torch.nextafter(mids, torch.tensor(0.0)), torch.nextafter(mids, torch.tensor(1e9)),
                   torch.tensor([0.0, -0.0, 1e-30, -1e-30, 1e6, -1e6, float(mag[-1]) * 1.0001])]).float().contiguous()
    expect = quantize_rtn(q[None, :], torch.ones(1), e, m)[0].numpy()
    got = np.zeros(q.numel(), np.uint8)
    harness.harness_quantize.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    harness.harness_quantize.restype = None
    harness.harness_quantize(e, m, ctypes.c_void_p(q.numpy().ctypes.data), q.numel(), ctypes.c_void_p(got.ctypes.data))
    assert np.array_equal(got, expect)
