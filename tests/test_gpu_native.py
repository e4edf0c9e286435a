"""The layer on the tensor cores' own six-bit inputs (fp6b200_linear_native): the weight re-layout bit for bit against
a numpy restatement, the layer against the oracle (tolerances of the linear layer) and against the fp16-pattern kernel
(both accumulate exact products in fp32, so they agree far inside the tolerance), with every path a tile can take to
memory and the fused epilogues."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_FRO = 2e-3
ROW_MAX = 1e-2
NATIVE_FORMATS = ((3, 2), (2, 3), (2, 2), (3, 1), (2, 1))   # the last three are widened to e2m3 / e3m2 / e2m3 codes


def _native_from_codes(codes: np.ndarray) -> np.ndarray:
    """uint8 codes [OC, IC] -> the tile layout: tiles of 128 rows x 128 K in (row tile, K tile) order, each row of a tile
    96 bytes, code i of the row at bits 6 i .. 6 i + 5 (little endian); K padded with code 0 to a multiple of 128."""
    oc, ic = codes.shape
    kt = (ic + 127) // 128
    padded = np.zeros((oc, kt * 128), dtype=np.uint64)
    padded[:, :ic] = codes
    tiles = padded.reshape(oc // 128, 128, kt, 128).transpose(0, 2, 1, 3)          # [mt, kt, row, k]
    groups = tiles.reshape(oc // 128, kt, 128, 8, 16)                              # 16 codes -> 12 bytes
    out = np.zeros(groups.shape[:4] + (12,), dtype=np.uint8)
    lo = np.zeros(groups.shape[:4], dtype=np.uint64)
    hi = np.zeros(groups.shape[:4], dtype=np.uint64)
    for i in range(16):
        bit = 6 * i
        if bit < 64:
            lo |= (groups[..., i] << np.uint64(bit)) & np.uint64(0xFFFFFFFFFFFFFFFF)
            if bit + 6 > 64:
                hi |= groups[..., i] >> np.uint64(64 - bit)
        else:
            hi |= groups[..., i] << np.uint64(bit - 64)
    for b in range(8):
        out[..., b] = (lo >> np.uint64(8 * b)) & np.uint64(0xFF)
    for b in range(4):
        out[..., 8 + b] = (hi >> np.uint64(8 * b)) & np.uint64(0xFF)
    return out.reshape(-1)


@pytest.mark.parametrize("e,m", NATIVE_FORMATS)
@pytest.mark.parametrize("oc,ic", [(256, 128), (512, 320), (1024, 1024)])
def test_repack_matches_numpy(e, m, oc, ic):
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer, unpack_codes
    w, _ = random_codes_layer(oc, ic, e, m, seed=oc + ic)
    packed = f.weight_prepacking_eXmY_cpu(e, m, w.cuda())
    native = f.native_repack(e, m, packed)
    assert native.dtype == torch.uint8 and native.numel() == (oc // 128) * ((ic + 127) // 128) * 128 * 96
    codes = unpack_codes(w, e, m).numpy().astype(np.uint32)
    bw = 1 + e + m
    six = ((codes >> (bw - 1)) << 5) | ((codes & ((1 << (bw - 1)) - 1)) << (6 - bw))      # sign kept, mantissa extended by zeros
    expect = _native_from_codes(six.astype(np.uint8))
    assert np.array_equal(native.cpu().numpy(), expect)


def _problem(oracle_mod, e, m, oc, ic, bs, seed, act_scale=1.0):
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer
    w, s = random_codes_layer(oc, ic, e, m, seed, scale_lo=0.005, scale_hi=0.02)
    x = (torch.randn(bs, ic, generator=torch.Generator().manual_seed(seed + 1)) * act_scale).half()
    packed = f.weight_prepacking_eXmY_cpu(e, m, w.cuda())
    native = f.native_repack(e, m, packed)
    truth = oracle_mod.linear(x.numpy(), w.numpy(), s.numpy(), e, m)
    return packed, native, s.cuda(), x.cuda(), truth


def _close(oracle_mod, y, truth):
    import fp6_llm_b200 as f
    assert f.device_status() == 0
    res = oracle_mod.check_tolerance(y.float().cpu().numpy(), truth.astype(np.float32))
    assert res["rel_fro"] <= REL_FRO and res["max_row_rel"] <= ROW_MAX, res
    return res


# every MMA width (tokens <= 4, 8, 16, 32, 64), whole tiles only (few tiles), stream-K remainder with a fix-up, K not a
# multiple of 128, long K
SHAPES = [(512, 1024, 1), (512, 1024, 4), (768, 2048, 7), (4096, 2048, 12), (1536, 4096, 16), (2048, 1088, 23), (1024, 8192, 32),
          (4096, 4096, 40), (19200, 1024, 64), (256, 64, 3), (256, 28672, 5)]


@pytest.mark.parametrize("oc,ic,bs", SHAPES)
@pytest.mark.parametrize("e,m", NATIVE_FORMATS)
def test_native_linear_matches_oracle_and_fp16_path(oracle_mod, e, m, oc, ic, bs):
    import fp6_llm_b200 as f
    packed, native, s, x, truth = _problem(oracle_mod, e, m, oc, ic, bs, seed=oc + ic + bs)
    y = f.linear_forward_native(e, m, x, native, s)
    assert y.shape == (bs, oc) and y.dtype == torch.float16
    _close(oracle_mod, y, truth)
    # against the fp16-pattern kernel: same exact products, fp32 sums in another order, one rounding to fp16 each
    ref = f.linear_forward_eXmY_cuda(e, m, x, packed, s, 0).float()
    diff = (y.float() - ref).abs().max().item()
    assert diff <= 2e-3 * ref.abs().max().item() + 1e-6, diff


@pytest.mark.parametrize("act_scale", [1e-4, 30.0, 3000.0])
def test_activation_range_is_split_exactly(oracle_mod, act_scale):
    """Small activations (fp16 subnormals among them) and large ones: the four planes carry every bit."""
    import fp6_llm_b200 as f
    packed, native, s, x, truth = _problem(oracle_mod, 3, 2, 512, 1024, 9, seed=77, act_scale=act_scale)
    y = f.linear_forward_native(3, 2, x, native, s)
    ref = f.linear_forward_eXmY_cuda(3, 2, x, packed, s, 0)
    assert torch.isfinite(y).all()
    _close(oracle_mod, y, truth)
    assert (y.float() - ref.float()).abs().max().item() <= 2e-3 * ref.float().abs().max().item() + 1e-7


def test_integer_valued_problem_is_exact():
    """Codes and activations whose products and sums are small integers: the result must be exact, whatever the order."""
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import pack_codes
    oc, ic, bs = 512, 640, 6
    gen = torch.Generator().manual_seed(5)
    # e3m2 codes of 0, 1, 2, 3, 4 and their negatives
    table = torch.tensor([0b000000, 0b001100, 0b010000, 0b010010, 0b010100, 0b101100, 0b110000, 0b110010, 0b110100], dtype=torch.uint8)
    values = torch.tensor([0.0, 1.0, 2.0, 3.0, 4.0, -1.0, -2.0, -3.0, -4.0])
    idx = torch.randint(0, 9, (oc, ic), generator=gen)
    w = pack_codes(table[idx], 3, 2)
    x = torch.randint(-4, 5, (bs, ic), generator=gen).half()
    s = torch.ones(oc, dtype=torch.float16)
    native = f.native_repack(3, 2, f.weight_prepacking_eXmY_cpu(3, 2, w.cuda()))
    y = f.linear_forward_native(3, 2, x.cuda(), native, s.cuda())
    truth = x.double() @ values[idx].double().T
    assert truth.abs().max() < 2048                    # exactly representable in fp16
    assert torch.equal(y.cpu().double(), truth)


@pytest.mark.parametrize("oc,ic,bs", [(512, 1024, 8), (4096, 2048, 12), (1536, 4096, 40)])
def test_native_epilogues(oracle_mod, oc, ic, bs):
    import fp6_llm_b200 as f
    packed, native, s, x, plain = _problem(oracle_mod, 3, 2, oc, ic, bs, seed=oc + bs + 3)
    bias = (torch.randn(oc, generator=torch.Generator().manual_seed(9)) * 2).half()
    y = f.linear_forward_native(3, 2, x, native, s, bias.cuda(), f.ACT_NONE)
    _close(oracle_mod, y, plain + bias.float().numpy()[None, :])
    pre = plain + bias.float().numpy()[None, :]
    gate, up = pre[:, 0::2], pre[:, 1::2]
    y = f.linear_forward_native(3, 2, x, native, s, bias.cuda(), f.ACT_SILU_MUL)
    assert y.shape == (bs, oc // 2)
    _close(oracle_mod, y, gate / (1.0 + np.exp(-gate)) * up)


def test_native_rejects_what_it_does_not_take():
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer
    assert not f.native_supported(3, 3, 512, 1024, 8)            # not a format of the library
    assert not f.native_supported(3, 2, 512, 1024, 65)
    assert not f.native_supported(3, 2, 384, 1024, 8)
    w, s = random_codes_layer(512, 1024, 3, 2, seed=1)
    native = f.native_repack(3, 2, f.weight_prepacking_eXmY_cpu(3, 2, w.cuda()))
    with pytest.raises(ValueError):
        f.linear_forward_native(3, 2, torch.zeros(65, 1024, dtype=torch.float16, device="cuda"), native, s.cuda())
    with pytest.raises(ValueError):
        f.linear_forward_native(3, 2, torch.zeros(8, 2048, dtype=torch.float16, device="cuda"), native, s.cuda())
    w5, _ = random_codes_layer(384, 1024, 2, 2, seed=1)
    with pytest.raises(ValueError):
        f.native_repack(2, 2, f.weight_prepacking_eXmY_cpu(2, 2, w5.cuda()))      # OC % 256 != 0


def test_native_repeated_calls_on_one_stream_share_the_scratch(oracle_mod):
    """Back-to-back calls of different shapes reuse one scratch buffer (activation planes, stream-K slots): each result
    must still be that of a call alone."""
    import fp6_llm_b200 as f
    probs = [_problem(oracle_mod, 3, 2, oc, ic, bs, seed=oc + bs) for oc, ic, bs in [(4096, 2048, 12), (512, 4096, 3), (1536, 1024, 33)]]
    alone = [f.linear_forward_native(3, 2, x, native, s).clone() for _, native, s, x, _ in probs]
    torch.cuda.synchronize()
    again = []
    for _ in range(3):
        again = [f.linear_forward_native(3, 2, x, native, s) for _, native, s, x, _ in probs]
    torch.cuda.synchronize()
    for a, b in zip(alone, again):
        assert torch.equal(a, b)
    assert f.device_status() == 0
