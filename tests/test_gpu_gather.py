"""The sharded layer with the exchange fused in (fp6b200_linear_gather): the kernel stores its rows into the output
buffer of every rank and ends with an arrival barrier between the GPUs.

On one GPU the two "ranks" are two sets of local buffers and the calls are made one after the other; the word a peer
would write is put there by the test beforehand, so no kernel ever waits for another launch.  The real two-process,
two-GPU run is at the bottom (skipped on a one-GPU box)."""
import ctypes
import os
import subprocess
import sys
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _layer(oc, ic, seed):
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer
    w, s = random_codes_layer(oc, ic, 3, 2, seed, scale_lo=0.01, scale_hi=0.1)
    return w.cuda(), s.cuda()


def _ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _gather_call(L, rank, world, packed, scale, x, outs, flags, epoch, oc, r0, split_k=0):
    import fp6_llm_b200 as f
    rows, bs, ic = packed.shape[0], x.shape[0], x.shape[1]
    nbytes = L.fp6b200_workspace_bytes(rows, bs, ic, split_k)
    ws = torch.empty(max(nbytes, 4) // 4, dtype=torch.float32, device="cuda")
    return L.fp6b200_linear_gather(3, 2, None, packed.data_ptr(), scale.data_ptr(), x.data_ptr(), _ptrs(outs), _ptrs(flags),
                                   epoch.data_ptr(), world, rank, oc, r0, rows, bs, ic, ws.data_ptr(), split_k)


@pytest.mark.parametrize("oc,ic,bs", [(1024, 512, 3), (4096, 4096, 8), (2560, 1024, 40), (512, 256, 130)])
def test_two_ranks_emulated_on_one_gpu(native_lib, oc, ic, bs):
    import fp6_llm_b200 as f
    from fp6_llm_b200.sharding import plan_rows
    L = native_lib
    w, s = _layer(oc, ic, seed=oc + bs)
    x = torch.randn(bs, ic, generator=torch.Generator().manual_seed(7)).half().cuda()
    plan = plan_rows(oc, 2)
    outs = [torch.full((bs, oc), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    epochs = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(2)]
    shards = []
    for rank, (r0, r1) in enumerate(plan):
        packed = f.weight_prepacking_cpu(w[r0:r1].contiguous())
        shards.append((packed, s[r0:r1].contiguous()))
    for call in range(1, 3):                                        # two rounds: the call counter advances on the device
        for o in outs:
            o.fill_(float("nan"))
        for rank, (r0, r1) in enumerate(plan):
            flags[rank][1 - rank] = call                            # what the other rank's barrier would have written
            rc = _gather_call(L, rank, 2, shards[rank][0], shards[rank][1], x, outs, flags, epochs[rank], oc, r0)
            assert rc == 0, L.fp6b200_error_string(rc)
            assert f.device_status() == 0
            expect = f.linear_forward_cuda(x, shards[rank][0], shards[rank][1], 0)      # same shard, plain entry point
            for o in outs:
                assert torch.equal(o[:, r0:r1], expect)             # same kernel, same plan: identical bits, in both buffers
            if rank == 0:
                assert torch.isnan(outs[0][:, plan[1][0]:]).all()   # rows of the other shard were not touched
            assert int(epochs[rank].item()) == call
            assert int(flags[1 - rank][rank].item()) == call        # the peer was told
            assert int(flags[rank][rank].item()) == call
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("oc,ic,bs", [(1024, 512, 3), (4096, 4096, 8), (2560, 1024, 30)])
def test_two_ranks_emulated_on_one_gpu_native_path(native_lib, oc, ic, bs):
    """The same exchange from the kernel that feeds the six-bit codes straight to the tensor cores."""
    import fp6_llm_b200 as f
    from fp6_llm_b200.sharding import plan_rows
    L = native_lib
    w, s = _layer(oc, ic, seed=oc + bs + 1)
    x = torch.randn(bs, ic, generator=torch.Generator().manual_seed(7)).half().cuda()
    plan = plan_rows(oc, 2)
    outs = [torch.full((bs, oc), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    epochs = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(2)]
    ws = torch.empty(L.fp6b200_native_workspace_bytes(bs, ic), dtype=torch.uint8, device="cuda")
    for rank, (r0, r1) in enumerate(plan):
        native = f.native_repack(3, 2, f.weight_prepacking_cpu(w[r0:r1].contiguous()))
        scale = s[r0:r1].contiguous()
        flags[rank][1 - rank] = 1                                   # what the other rank's barrier would have written
        rc = L.fp6b200_linear_native_gather(3, 2, None, native.data_ptr(), scale.data_ptr(), x.data_ptr(), _ptrs(outs), _ptrs(flags),
                                            epochs[rank].data_ptr(), 2, rank, oc, r0, r1 - r0, bs, ic, ws.data_ptr())
        assert rc == 0, L.fp6b200_error_string(rc)
        assert f.device_status() == 0
        expect = f.linear_forward_native(3, 2, x, native, scale)
        for o in outs:
            assert torch.equal(o[:, r0:r1], expect)
        assert int(flags[1 - rank][rank].item()) == 1
    assert torch.equal(outs[0], outs[1]) and not torch.isnan(outs[0]).any()


def test_barrier_gives_up_when_a_peer_never_arrives(native_lib):
    """The wait for a peer is bounded: with a flag nobody sets the call still returns, the status word says so
    (code 10) and the device stays usable."""
    import fp6_llm_b200 as f
    L = native_lib
    w, s = _layer(512, 256, seed=11)
    x = torch.randn(4, 256, generator=torch.Generator().manual_seed(1)).half().cuda()
    packed = f.weight_prepacking_cpu(w[:256].contiguous())
    outs = [torch.zeros((4, 512), dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    rc = _gather_call(L, 0, 2, packed, s[:256].contiguous(), x, outs, flags, epoch, 512, 0)
    assert rc == 0
    assert f.device_status() == 10
    assert 1.5 < time.perf_counter() - t0 < 10.0
    expect = f.linear_forward_cuda(x, packed, s[:256].contiguous(), 0)     # the device still works, and the rows were stored
    assert f.device_status() == 0
    assert torch.equal(outs[1][:, :256], expect)


def test_gather_rejects_bad_arguments(native_lib):
    import fp6_llm_b200 as f
    L = native_lib
    w, s = _layer(512, 256, seed=12)
    x = torch.randn(4, 256).half().cuda()
    packed = f.weight_prepacking_cpu(w[:256].contiguous())
    outs = [torch.zeros((4, 512), dtype=torch.float16, device="cuda")]
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda")]
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert _gather_call(L, 0, 1, packed, s[:256].contiguous(), x, outs, flags, epoch, 512, 384) == 1      # rows do not fit
    assert _gather_call(L, 1, 1, packed, s[:256].contiguous(), x, outs, flags, epoch, 512, 0) == 1        # rank >= world
    assert _gather_call(L, 0, 1, packed, s[:256].contiguous(), x, outs, flags, epoch, 512, 0, split_k=2) == 1
    assert _gather_call(L, 0, 1, packed, s[:256].contiguous(), x, outs, flags, epoch, 512, 0) == 0        # world of one: plain layer
    assert f.device_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_per_gpu():
    """One process per GPU (2, 4 or 8 of them): symmetric-memory buffers, peer stores over NVLink, the barrier
    between real ranks."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    ranks = max(n for n in (2, 4, 8) if n <= torch.cuda.device_count())
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(ranks), "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "gather_worker.py")]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "gather worker ok" in done.stdout
