"""GPU parity of the weight-format kernels, through the C interface: bit-exact against the CPU oracle, the
reference-made fixtures and the known-answer words."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import ALL_FORMATS, FORMATS, kat_ones, load_golden, random_unpacked

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(a).cuda()


def _prepack_dev(lib, w_np, e, m):
    rows = w_np.shape[0]
    cols = w_np.shape[1] * 32 // (1 + e + m)
    src = _dev(w_np)
    dst = torch.empty_like(src)
    rc = lib.fp6b200_prepack(e, m, None, src.data_ptr(), dst.data_ptr(), rows, cols)
    assert rc == 0, lib.fp6b200_error_string(rc)
    torch.cuda.synchronize()
    return dst.cpu().numpy()


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_prepack_golden(native_lib, e, m):
    for name in (f"prepack_dequant_e{e}m{m}.npz", f"all_codes_e{e}m{m}.npz"):
        g = load_golden(name)
        assert np.array_equal(_prepack_dev(native_lib, g["unpacked"], e, m), g["packed"])


@pytest.mark.parametrize("e,m", ALL_FORMATS)
@pytest.mark.parametrize("rows,cols", [(64, 64), (256, 128), (192, 320), (1024, 4096), (4096, 11008)])
def test_prepack_random_vs_oracle(native_lib, oracle_mod, e, m, rows, cols):
    rng = np.random.default_rng(rows + 7 * cols + e)
    w = random_unpacked(rng, rows, cols, e, m)
    assert np.array_equal(_prepack_dev(native_lib, w, e, m), oracle_mod.prepack(w, e, m))


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_prepack_host_entry_and_in_place(native_lib, oracle_mod, e, m):
    rng = np.random.default_rng(9)
    w = random_unpacked(rng, 256, 256, e, m)
    expect = oracle_mod.prepack(w, e, m)
    out = np.zeros_like(w)
    assert native_lib.fp6b200_prepack_host(e, m, out.ctypes.data, w.ctypes.data, 256, 256) == 0
    assert np.array_equal(out, expect)
    buf = w.copy()                                   # the reference's tests pack in place (tests/cpp/kernel_test_fp6.cu:27)
    assert native_lib.fp6b200_prepack_host(e, m, buf.ctypes.data, buf.ctypes.data, 256, 256) == 0
    assert np.array_equal(buf, expect)


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_python_prepack_operator_cpu_and_cuda_tensors(oracle_mod, e, m):
    import fp6_llm_b200 as f
    rng = np.random.default_rng(10)
    w = torch.from_numpy(random_unpacked(rng, 512, 128, e, m))
    expect = torch.from_numpy(oracle_mod.prepack(w.numpy(), e, m))
    got_cpu = f.weight_prepacking_eXmY_cpu(e, m, w)
    assert not got_cpu.is_cuda and torch.equal(got_cpu, expect)
    got_gpu = f.weight_prepacking_eXmY_cpu(e, m, w.cuda())
    assert got_gpu.is_cuda and torch.equal(got_gpu.cpu(), expect)
    if (e, m) == (3, 2):
        assert torch.equal(f.weight_prepacking_cpu(w), expect)
    with pytest.raises(ValueError):
        f.weight_prepacking_eXmY_cpu(e, m, w[:128])          # OC % 256
    with pytest.raises(ValueError):
        f.weight_prepacking_eXmY_cpu(4, 3, w)


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_dequant_unpacked_bit_exact(native_lib, oracle_mod, e, m):
    import fp6_llm_b200 as f
    g = load_golden(f"prepack_dequant_e{e}m{m}.npz")
    got = f.weight_dequant_eXmY_cpu(e, m, torch.from_numpy(g["unpacked"]), torch.from_numpy(g["scale"]))
    assert np.array_equal(got.numpy().view(np.uint16), g["dequant"].view(np.uint16))
    rng = np.random.default_rng(3)
    rows, cols = 512, 1024
    w = random_unpacked(rng, rows, cols, e, m)
    scale = np.concatenate([rng.uniform(1e-7, 1e-4, 128), rng.uniform(1e-3, 4.0, 256), rng.uniform(1e3, 6e4, 128)]).astype(np.float16)
    got = f.weight_dequant_eXmY_cpu(e, m, torch.from_numpy(w).cuda(), torch.from_numpy(scale).cuda()).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), oracle_mod.dequant(w, scale, e, m).view(np.uint16))


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_dequant_packed_bit_exact(native_lib, oracle_mod, e, m):
    """prepacked -> fp16 with the GEMM's own unpack code equals the oracle's dequantisation of the unpacked
    weights, including rows whose 2^bias*scale overflows fp16 and subnormal results."""
    import fp6_llm_b200 as f
    rng = np.random.default_rng(4)
    rows, cols = 512, 320
    w = random_unpacked(rng, rows, cols, e, m)
    scale = np.concatenate([rng.uniform(1e-7, 1e-4, 128), rng.uniform(1e-3, 4.0, 256), rng.uniform(16.0, 2000.0, 128)]).astype(np.float16)
    packed = torch.from_numpy(oracle_mod.prepack(w, e, m)).cuda()
    got = f.dequant_packed_cuda(e, m, packed, torch.from_numpy(scale).cuda()).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), oracle_mod.dequant(w, scale, e, m).view(np.uint16))


@pytest.mark.parametrize("e,m", FORMATS)
def test_known_answer_words(native_lib, e, m):
    import fp6_llm_b200 as f
    w = torch.from_numpy(kat_ones(e, m, 256, 128))
    ones = torch.ones(256, dtype=torch.float16)
    assert torch.all(f.weight_dequant_eXmY_cpu(e, m, w, ones) == 1.0)
    packed = f.weight_prepacking_eXmY_cpu(e, m, w).cuda()
    assert torch.all(f.dequant_packed_cuda(e, m, packed, ones.cuda()) == 1.0)


def test_splitk_reduce_kernel(native_lib, oracle_mod):
    rng = np.random.default_rng(8)
    p = rng.standard_normal((7, 3, 512)).astype(np.float32)
    d = torch.from_numpy(p).cuda()
    out = torch.empty((3, 512), dtype=torch.float16, device="cuda")
    assert native_lib.fp6b200_splitk_reduce(None, out.data_ptr(), d.data_ptr(), 3 * 512, 7) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint16), oracle_mod.splitk_reduce(p).view(np.uint16))


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_quantize_prepack_matches_quantiser_then_packer(native_lib, e, m):
    """The fused kernel gives the bits of: round-to-nearest codes (formats.quantize_rtn) -> bit stream -> prepack.
    The inputs include exact ties between neighbouring magnitudes, values beyond the largest magnitude, signed
    zeros and fp16 subnormals."""
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import magnitudes, pack_codes, quantize_rtn
    gen = torch.Generator().manual_seed(7 + e)
    oc, ic = 512, 320
    w = (torch.randn(oc, ic, generator=gen) * 0.05).half()
    mag = magnitudes(e, m)
    scale = (w.float().abs().amax(dim=1) / mag[-1]).half()         # the usual per-row scale: nothing saturates by much
    mids = ((mag[:-1] + mag[1:]) * 0.5).half()                      # every midpoint is exact in fp16
    scale[:8] = 1.0                                                 # rows with scale 1: the values below are the quotients
    w[0, : mids.numel()] = mids
    w[1, : mids.numel()] = -mids
    w[2, :4] = torch.tensor([0.0, -0.0, 6.0e-8, -6.0e-8]).half()
    w[3, :4] = torch.tensor([1000.0, -1000.0, float(mag[-1]), -float(mag[-1])]).half()
    w[4, : mag.numel()] = mag.half()
    expect = f.weight_prepacking_eXmY_cpu(e, m, pack_codes(quantize_rtn(w, scale, e, m), e, m).cuda())
    got = f.quantize_prepack_cuda(w.cuda(), scale.cuda(), e, m)
    assert torch.equal(got, expect)
    # and the packed result dequantises to within half a step of the input
    back = f.dequant_packed_cuda(e, m, got, scale.cuda()).float().cpu()
    step = (mag[1:] - mag[:-1]).max()
    body = w[8:].float()
    assert ((back[8:] - body).abs() <= 0.51 * step * scale[8:].float()[:, None] + 1e-6).all()
