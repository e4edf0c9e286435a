"""The CPU oracle against the reference: its own compiled CPU code (oracle/_ref, when present), the known-answer
words of the reference's tests, and the committed fixtures that the reference code produced."""
import numpy as np
import pytest

from helpers import ALL_FORMATS, FORMATS, kat_ones, load_golden, random_unpacked


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_golden_prepack_and_dequant(oracle_mod, e, m):
    for name in (f"prepack_dequant_e{e}m{m}.npz", f"all_codes_e{e}m{m}.npz"):
        g = load_golden(name)
        assert np.array_equal(oracle_mod.prepack(g["unpacked"], e, m), g["packed"])
        got = oracle_mod.dequant(g["unpacked"], g["scale"], e, m)
        assert np.array_equal(got.view(np.uint16), g["dequant"].view(np.uint16))


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_all_codes_fixture_values(oracle_mod, e, m):
    """The all-codes fixture dequantises to the closed-form value table (scale 1)."""
    import torch
    from fp6_llm_b200.formats import code_values
    g = load_golden(f"all_codes_e{e}m{m}.npz")
    expect = code_values(e, m)[torch.from_numpy(g["codes"].astype(np.int64))].numpy()
    got = g["dequant"].astype(np.float32)
    assert np.array_equal(got, expect)
    assert np.array_equal(np.signbit(got), np.signbit(expect))
    assert set(np.unique(g["codes"])) == set(range(1 << (1 + e + m)))


@pytest.mark.parametrize("e,m", FORMATS)
def test_known_answer_all_ones(oracle_mod, e, m):
    w = kat_ones(e, m, 64, 128)
    assert np.all(oracle_mod.dequant(w, np.ones(64, np.float16), e, m) == np.float16(1.0))
    x = np.ones((3, 128), np.float16)
    assert np.all(oracle_mod.linear(x, w, np.ones(64, np.float16), e, m) == 128.0)


@pytest.mark.parametrize("e,m", ALL_FORMATS)
@pytest.mark.parametrize("rows,cols", [(64, 64), (256, 128), (192, 320)])
def test_against_compiled_reference(oracle_mod, e, m, rows, cols):
    if not oracle_mod.have_ref():
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(rows * 1000 + cols + e)
    w = random_unpacked(rng, rows, cols, e, m)
    assert np.array_equal(oracle_mod.prepack(w, e, m), oracle_mod.ref_prepack(w, e, m))
    # scales that exercise subnormal results, ordinary values and fp16 overflow
    scale = np.concatenate([rng.uniform(1e-7, 1e-4, rows // 4), rng.uniform(1e-3, 4.0, rows // 2),
                            rng.uniform(1e3, 6e4, rows - rows // 4 - rows // 2)]).astype(np.float16)
    a = oracle_mod.dequant(w, scale, e, m)
    b = oracle_mod.ref_dequant(w, scale, e, m)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))


def test_prepack_in_place_allowed(oracle_mod):
    rng = np.random.default_rng(5)
    w = random_unpacked(rng, 64, 64, 3, 2)
    expect = oracle_mod.prepack(w, 3, 2)
    buf = w.copy()
    rc = oracle_mod.lib().oracle_prepack(3, 2, buf.ctypes.data, buf.ctypes.data, 64, 64)
    assert rc == 0 and np.array_equal(buf, expect)


def test_rejects_bad_shapes_and_formats(oracle_mod):
    w = np.zeros((64, 12), np.int32)
    out = np.zeros_like(w)
    L = oracle_mod.lib()
    assert L.oracle_prepack(4, 3, out.ctypes.data, w.ctypes.data, 64, 64) == -1
    assert L.oracle_prepack(3, 2, out.ctypes.data, w.ctypes.data, 32, 64) == -1
    assert L.oracle_prepack(3, 2, out.ctypes.data, w.ctypes.data, 64, 32) == -1


def test_half_conversions_match_numpy(oracle_mod):
    L = oracle_mod.lib()
    rng = np.random.default_rng(0)
    xs = (rng.standard_normal(4000) * 10.0 ** rng.uniform(-9, 6, 4000)).astype(np.float32)
    xs = np.concatenate([xs, np.array([65519.99, 65520.0, 6e-8, 2.9802322e-8, 3e-8, 0.0, -0.0, 1e-10, 65504.0], np.float32)])
    with np.errstate(over="ignore"):
        for x in xs:
            assert L.oracle_float_to_half(float(x)) == int(np.float16(x).view(np.uint16))
    for h in range(0, 65536, 7):
        f = L.oracle_half_to_float(h)
        g = np.array([h], np.uint16).view(np.float16).astype(np.float32)[0]
        assert f == g or (np.isnan(f) and np.isnan(g))


def test_splitk_reduce_semantics(oracle_mod):
    rng = np.random.default_rng(1)
    p = rng.standard_normal((5, 4, 128)).astype(np.float32)
    acc = np.zeros((4, 128), np.float32)
    for s in range(5):
        acc = acc + p[s]
    assert np.array_equal(oracle_mod.splitk_reduce(p).view(np.uint16), acc.astype(np.float16).view(np.uint16))


def test_tolerance_checker(oracle_mod):
    y = np.ones((2, 8), np.float32)
    assert oracle_mod.check_tolerance(y, y)["ok"]
    bad = y.copy()
    bad[0, 0] = 1.02
    assert not oracle_mod.check_tolerance(bad, y)["ok"]
