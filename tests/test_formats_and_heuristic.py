import json
import os

import numpy as np
import pytest
import torch

from helpers import ALL_FORMATS, FORMATS, GOLDEN, KAT_ONES_E2M2, KAT_ONES_E3M2


def test_value_tables():
    from fp6_llm_b200.formats import magnitudes
    assert magnitudes(3, 2).tolist() == [0, .0625, .125, .1875, .25, .3125, .375, .4375, .5, .625, .75, .875, 1, 1.25, 1.5,
                                         1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 7, 8, 10, 12, 14, 16, 20, 24, 28]
    assert magnitudes(2, 2).tolist() == [0, .25, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 7]


def test_pack_codes_known_answer_words():
    from fp6_llm_b200.formats import pack_codes
    w = pack_codes(torch.full((2, 64), 0b001100, dtype=torch.uint8), 3, 2)
    assert w.view(torch.int32)[0, :3].numpy().astype(np.uint32).tolist() == list(KAT_ONES_E3M2)
    w = pack_codes(torch.full((2, 64), 0b00100, dtype=torch.uint8), 2, 2)
    assert w[0, :5].numpy().astype(np.uint32).tolist() == list(KAT_ONES_E2M2)


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_pack_unpack_roundtrip_and_values(oracle_mod, e, m):
    from fp6_llm_b200.formats import code_values, pack_codes, random_codes_layer, unpack_codes
    w, s = random_codes_layer(128, 192, e, m, seed=4, scale_lo=0.01, scale_hi=1.0)
    codes = unpack_codes(w, e, m)
    assert torch.equal(pack_codes(codes, e, m), w)
    expect = (code_values(e, m)[codes.long()] * s.float()[:, None]).half()
    got = torch.from_numpy(oracle_mod.dequant(w.numpy(), s.numpy(), e, m))
    assert torch.equal(got.view(torch.int16), expect.view(torch.int16))


@pytest.mark.parametrize("e,m", ALL_FORMATS)
def test_quantizer_nearest_even_and_saturation(e, m):
    from fp6_llm_b200.formats import magnitudes, quantize_rtn
    mag = magnitudes(e, m)
    one = torch.ones(1)
    assert quantize_rtn(mag[None, :].clone(), one, e, m)[0].tolist() == list(range(len(mag)))
    mid = (mag[:-1] + mag[1:]) / 2
    q = quantize_rtn(mid[None, :].clone(), one, e, m)[0]
    assert all(int(c) % 2 == 0 for c in q)                      # ties go to the even code
    big = torch.tensor([[mag[-1] * 3, -mag[-1] * 3, -0.0]])
    assert quantize_rtn(big, one, e, m)[0].tolist() == [len(mag) - 1, 2 * len(mag) - 1, len(mag)]


def test_reference_heuristic_reproduced():
    """HeuristicFuntion_SplitK / Num_Wave equal the reference's values (fixture made from fp6_llm/__init__.py:6-23)."""
    from fp6_llm_b200 import HeuristicFuntion_SplitK, Num_Wave
    cases = json.load(open(os.path.join(GOLDEN, "splitk_heuristic.json")))
    assert len(cases) > 100
    for c in cases:
        assert HeuristicFuntion_SplitK(c["M"], c["N"], c["SMs"]) == c["split_k"]
        assert Num_Wave(c["M"], c["N"], 3, c["SMs"]) == c["num_wave_k3"]


def test_b200_heuristic_is_sane(native_lib):
    from fp6_llm_b200 import heuristic_split_k_b200
    for M, N, K in [(4096, 8, 4096), (12288, 1, 4096), (22016, 32, 4096), (4096, 128, 11008), (57344, 2048, 8192)]:
        k = heuristic_split_k_b200(M, N, K)
        assert 1 <= k <= K // 64
    assert heuristic_split_k_b200(57344, 2048, 8192) == 1        # plenty of tiles: no split
    assert heuristic_split_k_b200(4096, 1, 4096) > 1             # 32 tiles on 148 SMs: split
