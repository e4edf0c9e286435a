"""The entry point for callers that cannot allocate device memory (pre-reserved pools, fixed memory
budgets): it must give the same output as the ordinary entry point, on two calls in a row (the built-in scratch array
keeps the first call's contents when the second one runs), and refuse problems its fixed scratch cannot hold."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(oc, ic, bs, seed, oracle_mod=None):
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer
    w, s = random_codes_layer(oc, ic, 3, 2, seed, scale_lo=0.01, scale_hi=0.1)
    packed = f.weight_prepacking_cpu(w.cuda())
    x = torch.randn(bs, ic, generator=torch.Generator().manual_seed(seed + 1)).half()
    truth = oracle_mod.linear(x.numpy(), w.numpy(), s.numpy(), 3, 2) if oracle_mod is not None else None
    return packed, s.cuda(), x.cuda(), truth


def test_static_scratch_matches_workspace_entry(native_lib, oracle_mod):
    import fp6_llm_b200 as f
    L = native_lib
    # two different problems back to back: 32 tiles dealt over all SMs (every tile goes through the scratch), then a
    # shape whose remainder tiles do
    for oc, ic, bs, seed in ((4096, 2048, 8, 3), (1536, 4096, 40, 4)):
        packed, s, x, truth = _problem(oc, ic, bs, seed, oracle_mod)
        expect = f.linear_forward_cuda(x, packed, s, 0)                   # ordinary entry point, caller-owned workspace
        for _ in range(2):
            out = torch.full((bs, oc), float("nan"), dtype=torch.float16, device="cuda")
            rc = L.fp6b200_linear_static_scratch(3, 2, None, packed.data_ptr(), s.data_ptr(), x.data_ptr(), out.data_ptr(),
                                                 oc, bs, ic)
            assert rc == 0, L.fp6b200_error_string(rc)
            assert f.device_status() == 0
            # same kernel, same decomposition, same summation order: the tolerance of the linear-layer tests is ample
            err = (out.float() - expect.float()).norm() / expect.float().norm()
            assert err.item() <= 2e-3
            assert torch.equal(out, expect)
            # and against the oracle itself (reference dequantisation + fp32 matmul), with the linear layer's tolerances
            res = oracle_mod.check_tolerance(out.float().cpu().numpy(), truth)
            assert res["rel_fro"] <= 2e-3 and res["max_row_rel"] <= 1e-2, res


def test_static_scratch_refuses_oversized_problems(native_lib):
    L = native_lib
    packed, s, x, _ = _problem(256, 256, 4, 5)
    assert L.fp6b200_static_scratch_bytes() == 10 << 20
    big_n = 4096                                                          # 256-wide tiles: far more scratch than the array
    assert L.fp6b200_workspace_bytes(256, big_n, 256, 0) > L.fp6b200_static_scratch_bytes()
    out = torch.empty(4, 256, dtype=torch.float16, device="cuda")
    rc = L.fp6b200_linear_static_scratch(3, 2, None, packed.data_ptr(), s.data_ptr(), x.data_ptr(), out.data_ptr(), 256, big_n, 256)
    assert rc == 1                                                        # cudaErrorInvalidValue, nothing launched
