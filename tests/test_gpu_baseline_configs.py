"""GPU parity of the linear layer on the shapes and batch sizes the benchmark workloads are quoted on.

Against the oracle (reference dequantisation + fp32 matmul) on row slices that keep the FULL K and the full batch-size
set of every workload: LLaMA-2-7B FP6 (K 4096 / 11008), LLaMA-2-13B FP5 (K 5120 / 13824, explicit split-K 1/2/4/8 and
the library's own decomposition), LLaMA-2-70B FP6 (K 8192 / 28672, batch 1..128) and the prefill batches 512..2048.
At the FULL layer shapes the oracle is too slow, so every (layer, batch) pair of the 70B workloads is checked per block
of 32 output channels against an fp32 matmul on the GPU-dequantised weights (that dequantiser is bit-exact against the
oracle, see test_gpu_formats.py).  Tolerances as in test_gpu_linear.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_FRO = 2e-3
ROW_MAX = 1e-2


def _oracle_case(oracle_mod, e, m, oc, ic, bs, seed, scale_lo=None, scale_hi=None, act_scale=1.0):
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer, synth_layer
    if scale_lo is None:
        w, s = synth_layer(oc, ic, e, m, seed)
    else:
        w, s = random_codes_layer(oc, ic, e, m, seed, scale_lo=scale_lo, scale_hi=scale_hi)
    x = (torch.randn(bs, ic, generator=torch.Generator().manual_seed(seed + 1)) * act_scale).half()
    packed = f.weight_prepacking_eXmY_cpu(e, m, w.cuda())
    truth = oracle_mod.linear(x.numpy(), w.numpy(), s.numpy(), e, m)
    return packed, s.cuda(), x.cuda(), truth


def _check(oracle_mod, y, truth):
    import fp6_llm_b200 as f
    assert f.device_status() == 0, "a GEMM CTA timed out"
    res = oracle_mod.check_tolerance(y.float().cpu().numpy(), truth)
    assert res["rel_fro"] <= REL_FRO and res["max_row_rel"] <= ROW_MAX, res


@pytest.mark.parametrize("oc,ic", [(1024, 4096), (768, 11008)])
@pytest.mark.parametrize("bs", [1, 8, 32, 128])
def test_llama2_7b_fp6_slices(oracle_mod, oc, ic, bs):
    import fp6_llm_b200 as f
    packed, s, x, truth = _oracle_case(oracle_mod, 3, 2, oc, ic, bs, seed=oc + bs)
    _check(oracle_mod, f.linear_forward_cuda(x, packed, s, 0), truth)


@pytest.mark.parametrize("oc,ic", [(1280, 5120), (512, 13824)])
@pytest.mark.parametrize("bs", [1, 16, 64])
@pytest.mark.parametrize("split_k", [1, 2, 4, 8, 0])
def test_llama2_13b_fp5_slices_every_split(oracle_mod, oc, ic, bs, split_k):
    import fp6_llm_b200 as f
    packed, s, x, truth = _oracle_case(oracle_mod, 2, 2, oc, ic, bs, seed=ic + bs)
    _check(oracle_mod, f.linear_forward_eXmY_cuda(2, 2, x, packed, s, split_k), truth)


@pytest.mark.parametrize("oc,ic", [(768, 8192), (512, 28672)])
@pytest.mark.parametrize("bs", [1, 4, 16, 64, 128])
def test_llama2_70b_fp6_slices(oracle_mod, oc, ic, bs):
    import fp6_llm_b200 as f
    packed, s, x, truth = _oracle_case(oracle_mod, 3, 2, oc, ic, bs, seed=ic + bs)
    _check(oracle_mod, f.linear_forward_cuda(x, packed, s, 0), truth)


@pytest.mark.parametrize("oc,ic", [(512, 8192), (256, 28672)])
@pytest.mark.parametrize("bs", [512, 1024, 2048])
def test_llama2_70b_prefill_slices(oracle_mod, oc, ic, bs):
    import fp6_llm_b200 as f
    packed, s, x, truth = _oracle_case(oracle_mod, 3, 2, oc, ic, bs, seed=ic + bs)
    _check(oracle_mod, f.linear_forward_cuda(x, packed, s, 0), truth)


@pytest.mark.parametrize("e,m", [(3, 2), (2, 2)])
@pytest.mark.parametrize("bs,split_k", [(5, 0), (40, 1), (130, 3)])
def test_scales_beyond_the_fp16_range_of_scale_times_bias(oracle_mod, e, m, bs, split_k):
    """Row scales in (16, 2000): scale * 2^12 (e3m2) or scale * 2^14 (e2m2) does not fit fp16, so a kernel that folded
    the bias into the scale in fp16 would overflow; the epilogue multiplies in fp32.  Small activations keep the
    outputs inside fp16."""
    import fp6_llm_b200 as f
    top = 2000.0 if e == 3 else 8000.0   # the largest dequantised weight (28 * 2000, 7 * 8000) still fits fp16
    packed, s, x, truth = _oracle_case(oracle_mod, e, m, 512, 1024, bs, seed=bs, scale_lo=16.0, scale_hi=top, act_scale=1e-3)
    assert float(s.float().min()) >= 16.0
    _check(oracle_mod, f.linear_forward_eXmY_cuda(e, m, x, packed, s, split_k), truth)


@pytest.mark.parametrize("e,m", [(2, 1), (3, 1), (2, 3)])
@pytest.mark.parametrize("oc,ic,bs,split_k", [(512, 1024, 1, 0), (768, 4096, 16, 0), (512, 2048, 40, 3), (256, 8192, 130, 0), (512, 1024, 300, 1)])
def test_other_formats_of_the_reference_templates(oracle_mod, e, m, oc, ic, bs, split_k):
    """e2m1 (4-bit), e3m1 (5-bit) and e2m3 (6-bit): formats the reference's packer and dequantiser templates cover although
    its GEMM launcher does not; same oracle recipe, same tolerances, every tile width."""
    import fp6_llm_b200 as f
    packed, s, x, truth = _oracle_case(oracle_mod, e, m, oc, ic, bs, seed=oc + bs + e)
    _check(oracle_mod, f.linear_forward_eXmY_cuda(e, m, x, packed, s, split_k), truth)
    packed, s, x, truth = _oracle_case(oracle_mod, e, m, oc, ic, bs, seed=bs + e, scale_lo=0.01, scale_hi=0.1)   # uniformly random codes
    _check(oracle_mod, f.linear_forward_eXmY_cuda(e, m, x, packed, s, split_k), truth)


# ------------------------------------------------------------------------------------------------ full layer shapes
_FULL = {"qkv": (10240, 8192), "o": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}


@pytest.fixture(scope="module")
def full_layers():
    """Prepacked weights of the four LLaMA-2-70B layers, made once per test module on the GPU."""
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import synth_layer
    cache = {}

    def get(name):
        if name not in cache:
            cache.clear()                                  # one layer resident at a time
            oc, ic = _FULL[name]
            w, s = synth_layer(oc, ic, 3, 2, seed=len(name), device="cuda")
            cache[name] = (f.weight_prepacking_cpu(w), s)
            del w
        return cache[name]
    return get


def _blockwise_check(y, x, packed, s, rows_per_chunk=4096):
    """Every block of 32 output channels within the relative tolerance against fp32 matmul on the dequantised weights."""
    import fp6_llm_b200 as f
    oc, bs = packed.shape[0], x.shape[0]
    w16 = f.dequant_packed_cuda(3, 2, packed, s)
    xf = x.float()
    worst = 0.0
    for r0 in range(0, oc, rows_per_chunk):
        r1 = min(oc, r0 + rows_per_chunk)
        ref = xf @ w16[r0:r1].float().T                                   # [bs, rows]
        err = (y[:, r0:r1].float() - ref).T.reshape((r1 - r0) // 32, 32 * bs)
        refg = ref.T.reshape((r1 - r0) // 32, 32 * bs)
        worst = max(worst, float((err.norm(dim=1) / refg.norm(dim=1).clamp_min(1e-20)).max().item()))
        row = float(((y[:, r0:r1].float() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max().item())
        assert row <= ROW_MAX, (r0, row)
    assert worst <= REL_FRO, worst


@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
@pytest.mark.parametrize("bs", [1, 4, 16, 64, 128])
def test_full_llama2_70b_layers(full_layers, name, bs):
    import fp6_llm_b200 as f
    packed, s = full_layers(name)
    x = torch.randn(bs, _FULL[name][1], generator=torch.Generator(device="cuda").manual_seed(bs), device="cuda").half()
    y = f.linear_forward_cuda(x, packed, s, 0)
    assert f.device_status() == 0
    _blockwise_check(y, x, packed, s)


@pytest.mark.parametrize("name", ["gate_up", "down"])
@pytest.mark.parametrize("bs", [512, 1024, 2048])
def test_full_llama2_70b_prefill_layers(full_layers, name, bs):
    """Includes the 8192 x 28672 layer at batch 1024, the launch shape on which a ring-depth error once surfaced."""
    import fp6_llm_b200 as f
    packed, s = full_layers(name)
    x = torch.randn(bs, _FULL[name][1], generator=torch.Generator(device="cuda").manual_seed(bs), device="cuda").half()
    ys = [f.linear_forward_cuda(x, packed, s, 0) for _ in range(2)]      # back to back: the second launch follows a fix-up kernel
    assert f.device_status() == 0
    assert torch.equal(ys[0], ys[1])
    _blockwise_check(ys[1], x, packed, s)


# ------------------------------------------------------------------------------------------------ batched host entry
def test_batched_host_entry_matches_oracle(oracle_mod):
    """Several layers of different shapes and formats through fp6b200_linear_host_io_batch: pinned host activations in,
    host outputs back, copies pipelined around the kernels."""
    import fp6_llm_b200 as f
    calls, truths, outs = [], [], []
    for i, (e, m, oc, ic, bs) in enumerate(((3, 2, 1024, 1024, 24), (2, 2, 512, 2048, 3), (3, 2, 768, 4096, 130), (3, 2, 1024, 1024, 1),
                                             (3, 2, 16384, 1024, 130), (2, 2, 8192, 512, 300))):   # the last two: results of several MB
        packed, s, x, truth = _oracle_case(oracle_mod, e, m, oc, ic, bs, seed=40 + i)
        out = torch.empty(bs, oc, dtype=torch.float16).pin_memory()
        calls.append((e, m, x.cpu().pin_memory(), packed, s, out, 0))
        truths.append(truth)
        outs.append(out)
    # four times with the same buffers (the staging buffer, streams and events are reused), with other activations in the
    # same pinned buffers each time (scaled by a power of two, so the truth scales exactly)
    base = [c[2].clone() for c in calls]
    for factor in (1.0, 2.0, 0.5, 4.0):
        for c, b in zip(calls, base):
            c[2].copy_(b * factor)
        for o in outs:
            o.fill_(float("nan"))
        f.linear_forward_host_batch(calls)
        assert f.device_status() == 0
        for o, t in zip(outs, truths):
            _check(oracle_mod, o, t * factor)
    for c, b in zip(calls, base):
        c[2].copy_(b)
    # the same batch with the six-bit layers also given in the tile layout: the two small-batch e3m2 calls take the
    # tensor cores' own FP6 inputs, the others stay where they were
    with_native = [c + ((f.native_repack(c[0], c[1], c[3]),) if (c[0], c[1]) == (3, 2) else (None,)) for c in calls]
    for o in outs:
        o.fill_(float("nan"))
    f.linear_forward_host_batch(with_native)
    assert f.device_status() == 0
    for o, t in zip(outs, truths):
        _check(oracle_mod, o, t)
    with pytest.raises(ValueError):
        f.linear_forward_host_batch([(3, 2, calls[0][2][:, :512].contiguous(), calls[0][3], calls[0][4], calls[0][5], 0)])
