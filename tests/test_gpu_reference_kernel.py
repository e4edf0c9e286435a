"""The reference's own GPU kernel (fp6_llm/csrc/fp6_linear.cu, recompiled for sm_100a into oracle/_ref by oracle/Makefile,
target refgpu) run on the same prepacked weights as this library's kernels: both must agree within the tolerances of the
linear layer, and both with the oracle.  Skipped when that build is absent."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("e,m", [(3, 2), (2, 2)])
@pytest.mark.parametrize("oc,ic,bs,split_k", [(512, 1024, 8, 1), (1024, 4096, 3, 4), (768, 2048, 40, 2), (512, 1024, 130, 1)])
def test_reference_gpu_kernel_agrees(oracle_mod, e, m, oc, ic, bs, split_k):
    if not oracle_mod.have_ref_gpu():
        pytest.skip("oracle/_ref/libfp6_ref_gpu.so not built (needs a checkout of the reference)")
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer
    w, s = random_codes_layer(oc, ic, e, m, seed=oc + bs, scale_lo=0.005, scale_hi=0.02)
    x = torch.randn(bs, ic, generator=torch.Generator().manual_seed(3)).half()
    packed = f.weight_prepacking_eXmY_cpu(e, m, w.cuda())
    xd, sd = x.cuda(), s.cuda()
    out = torch.empty(bs, oc, dtype=torch.float16, device="cuda")
    ws = torch.empty(split_k * oc * bs, dtype=torch.float32, device="cuda")
    rc = oracle_mod.ref_gpu().ref_gpu_linear(e, m, torch.cuda.current_stream().cuda_stream, packed.data_ptr(), sd.data_ptr(),
                                             xd.data_ptr(), out.data_ptr(), oc, bs, ic, ws.data_ptr(), split_k)
    torch.cuda.synchronize()
    assert rc == 0
    truth = oracle_mod.linear(x.numpy(), w.numpy(), s.numpy(), e, m)
    res = oracle_mod.check_tolerance(out.float().cpu().numpy(), truth)
    assert res["ok"], res                                   # the reference kernel against the oracle's recipe
    mine = f.linear_forward_eXmY_cuda(e, m, xd, packed, sd, 0)
    res = oracle_mod.check_tolerance(mine.float().cpu().numpy(), out.float().cpu().numpy().astype(np.float32))
    assert res["ok"], res                                   # this library against the reference kernel itself
    if f.native_supported(e, m, oc, ic, bs):
        nat = f.linear_forward_native(e, m, xd, f.native_repack(e, m, packed), sd)
        res = oracle_mod.check_tolerance(nat.float().cpu().numpy(), out.float().cpu().numpy().astype(np.float32))
        assert res["ok"], res
