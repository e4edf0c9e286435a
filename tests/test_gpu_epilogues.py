"""The fused epilogues of fp6b200_linear_ex (bias in fp32, silu(gate) * up on interleaved rows) against the oracle's
linear layer followed by the same arithmetic in fp32 on the CPU; every path a tile can take to memory: stored by the
GEMM, summed by the stream-K fix-up, summed by the split-K reduction.  Tolerances of the linear layer."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_FRO = 2e-3
ROW_MAX = 1e-2


def _problem(oracle_mod, e, m, oc, ic, bs, seed):
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer
    w, s = random_codes_layer(oc, ic, e, m, seed, scale_lo=0.005, scale_hi=0.02)
    x = torch.randn(bs, ic, generator=torch.Generator().manual_seed(seed + 1)).half()
    bias = (torch.randn(oc, generator=torch.Generator().manual_seed(seed + 2)) * 2).half()
    packed = f.weight_prepacking_eXmY_cpu(e, m, w.cuda())
    plain = oracle_mod.linear(x.numpy(), w.numpy(), s.numpy(), e, m)           # fp32 [bs, oc]
    return packed, s.cuda(), x.cuda(), bias, plain


def _close(oracle_mod, y, truth):
    import fp6_llm_b200 as f
    assert f.device_status() == 0
    res = oracle_mod.check_tolerance(y.float().cpu().numpy(), truth.astype(np.float32))
    assert res["rel_fro"] <= REL_FRO and res["max_row_rel"] <= ROW_MAX, res


# (oc, ic, bs, split_k): direct tiles only; stream-K with a fix-up; explicit split-K with the reduction kernel; wide tiles
SHAPES = [(512, 1024, 8, 1), (4096, 2048, 12, 0), (1536, 4096, 40, 0), (512, 2048, 33, 4), (768, 1024, 130, 0), (512, 1024, 300, 2)]


@pytest.mark.parametrize("oc,ic,bs,split_k", SHAPES)
@pytest.mark.parametrize("e,m", [(3, 2), (2, 2)])
def test_bias(oracle_mod, e, m, oc, ic, bs, split_k):
    import fp6_llm_b200 as f
    packed, s, x, bias, plain = _problem(oracle_mod, e, m, oc, ic, bs, seed=oc + bs)
    y = f.linear_forward_ex(e, m, x, packed, s, split_k, bias.cuda(), f.ACT_NONE)
    assert y.shape == (bs, oc)
    _close(oracle_mod, y, plain + bias.float().numpy()[None, :])
    # without bias the extended entry equals the plain one bit for bit
    assert torch.equal(f.linear_forward_ex(e, m, x, packed, s, split_k), f.linear_forward_eXmY_cuda(e, m, x, packed, s, split_k))


@pytest.mark.parametrize("oc,ic,bs,split_k", SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_silu_mul(oracle_mod, oc, ic, bs, split_k, with_bias):
    import fp6_llm_b200 as f
    packed, s, x, bias, plain = _problem(oracle_mod, 3, 2, oc, ic, bs, seed=oc + bs + 7)
    pre = plain + (bias.float().numpy()[None, :] if with_bias else 0.0)
    gate, up = pre[:, 0::2], pre[:, 1::2]                                       # rows 2c = gate, 2c+1 = up
    truth = gate / (1.0 + np.exp(-gate)) * up
    y = f.linear_forward_ex(3, 2, x, packed, s, split_k, bias.cuda() if with_bias else None, f.ACT_SILU_MUL)
    assert y.shape == (bs, oc // 2)
    _close(oracle_mod, y, truth)


def test_gate_up_module_matches_two_linears():
    """FPxGateUpLinear.from_linears: interleaves, quantises and packs two torch layers; its output equals silu(gate) * up
    computed in fp32 from the dequantised weights, and FPxLinear adds its bias inside the kernel."""
    import fp6_llm_b200 as f
    torch.manual_seed(5)
    gate = torch.nn.Linear(1024, 768, bias=True).cuda().half()
    up = torch.nn.Linear(1024, 768, bias=False).cuda().half()
    layer = f.FPxGateUpLinear.from_linears(gate, up)
    assert (layer.in_features, layer.out_features) == (1024, 768)
    x = torch.randn(4, 6, 1024, device="cuda").half()
    y = layer(x)
    assert y.shape == (4, 6, 768)
    w16 = f.dequant_packed_cuda(3, 2, layer.weight, layer.scales).float()
    pre = x.float().reshape(-1, 1024) @ w16.T + layer.bias.float()
    ref = torch.nn.functional.silu(pre[:, 0::2]) * pre[:, 1::2]
    err = (y.float().reshape(-1, 768) - ref).norm() / ref.norm()
    assert err.item() <= 2e-3 and f.device_status() == 0
    # close to the unquantised layers as well (6-bit weights: a few percent)
    full = torch.nn.functional.silu(gate(x).float()) * up(x).float()
    assert ((y.float() - full).norm() / full.norm()).item() < 0.08


def test_row_parallel_parts_sum_to_the_whole(oracle_mod):
    """IC-sharded layer on one GPU: the partial results of the column shards (each through the kernel, the bias on shard 0
    only) add up to the unsharded layer."""
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer
    from fp6_llm_b200.sharding import RowParallelFPxLinear, plan_cols, slice_unpacked_cols
    oc, ic, bs, world = 1024, 4096 + 64, 24, 3
    w, s = random_codes_layer(oc, ic, 3, 2, 21, scale_lo=0.005, scale_hi=0.02)
    x = torch.randn(bs, ic, generator=torch.Generator().manual_seed(3)).half()
    bias = torch.randn(oc, generator=torch.Generator().manual_seed(4)).half()
    plan = plan_cols(ic, world)
    total = torch.zeros(bs, oc, dtype=torch.float32, device="cuda")
    for r, (k0, k1) in enumerate(plan):
        packed = f.weight_prepacking_cpu(slice_unpacked_cols(w, 3, 2, k0, k1).cuda())
        layer = RowParallelFPxLinear(packed, s.cuda(), plan, r, 3, 2, bias=bias.cuda())
        total += layer.forward_local(x[:, k0:k1].contiguous().cuda()).float()
    truth = oracle_mod.linear(x.numpy(), w.numpy(), s.numpy(), 3, 2) + bias.float().numpy()[None, :]
    _close(oracle_mod, total, truth)
