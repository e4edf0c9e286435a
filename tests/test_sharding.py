"""OC-sharded layer: the shard planner, cutting a packed tensor, and the all-gather of column slabs run as two
gloo ranks on CPU (each rank's GEMM is played by the oracle; the collective and the slab assembly are the code
under test)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from helpers import FORMATS


def test_plan_rows():
    from fp6_llm_b200.sharding import plan_rows
    assert plan_rows(4096, 8) == [(i * 512, (i + 1) * 512) for i in range(8)]
    p = plan_rows(22016, 8)
    assert p[0] == (0, 2816) and p[-1] == (19456, 22016)
    assert all((b - a) % 256 == 0 for a, b in p) and all(p[i][1] == p[i + 1][0] for i in range(7))
    with pytest.raises(ValueError):
        plan_rows(4000, 2)
    with pytest.raises(ValueError):
        plan_rows(512, 4)


@pytest.mark.parametrize("e,m", FORMATS)
def test_shard_of_packed_equals_pack_of_shard(oracle_mod, e, m):
    from fp6_llm_b200.formats import random_codes_layer
    from fp6_llm_b200.sharding import plan_rows, shard_packed
    w, _ = random_codes_layer(1024, 128, e, m, seed=3)
    full = torch.from_numpy(oracle_mod.prepack(w.numpy(), e, m))
    for r0, r1 in plan_rows(1024, 3):
        expect = torch.from_numpy(oracle_mod.prepack(w[r0:r1].contiguous().numpy(), e, m))
        assert torch.equal(shard_packed(full, 128, e, m, r0, r1), expect)
        assert not torch.equal(full[r0:r1], expect)          # naive row slicing is wrong
    with pytest.raises(ValueError):
        shard_packed(full, 128, e, m, 32, 512)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, oc, ic, batch, result_dir):
    import torch.distributed as dist
    import oracle
    from fp6_llm_b200.formats import random_codes_layer
    from fp6_llm_b200.sharding import gather_columns, plan_rows
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w, s = random_codes_layer(oc, ic, 3, 2, seed=11, scale_lo=0.01, scale_hi=0.1)
        x = torch.randn(batch, ic, generator=torch.Generator().manual_seed(5)).half()
        plan = plan_rows(oc, world)
        r0, r1 = plan[rank]
        local = torch.from_numpy(oracle.linear(x.numpy(), w[r0:r1].contiguous().numpy(), s[r0:r1].numpy())).half()
        full = gather_columns(local, plan, rank)
        torch.save(full, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("oc", [512, 768])           # even shards, and 2+1 row units (padded gather)
def test_two_rank_gather_matches_unsharded(oracle_mod, tmp_path, oc):
    from fp6_llm_b200.formats import random_codes_layer
    ic, batch, world = 128, 5, 2
    mp.spawn(_rank_main, args=(world, _free_port(), oc, ic, batch, str(tmp_path)), nprocs=world, join=True)
    w, s = random_codes_layer(oc, ic, 3, 2, seed=11, scale_lo=0.01, scale_hi=0.1)
    x = torch.randn(batch, ic, generator=torch.Generator().manual_seed(5)).half()
    expect = torch.from_numpy(oracle_mod.linear(x.numpy(), w.numpy(), s.numpy())).half()
    for r in range(world):
        got = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        assert got.shape == (batch, oc)
        assert torch.equal(got, expect)


# ------------------------------------------------------------------------------------------------ IC-sharded (row-parallel)
def test_plan_cols_and_column_slices(oracle_mod):
    from fp6_llm_b200.formats import random_codes_layer, unpack_codes
    from fp6_llm_b200.sharding import plan_cols, slice_unpacked_cols
    assert plan_cols(8192, 8) == [(i * 1024, (i + 1) * 1024) for i in range(8)]
    p = plan_cols(28672, 8)
    assert all((b - a) % 64 == 0 for a, b in p) and p[0][0] == 0 and p[-1][1] == 28672
    assert plan_cols(11008, 3) == [(0, 3712), (3712, 7360), (7360, 11008)]
    with pytest.raises(ValueError):
        plan_cols(100, 2)
    for e, m in FORMATS:
        w, _ = random_codes_layer(256, 320, e, m, seed=2)
        codes = unpack_codes(w, e, m)
        for k0, k1 in plan_cols(320, 2):
            assert torch.equal(unpack_codes(slice_unpacked_cols(w, e, m, k0, k1), e, m), codes[:, k0:k1])
        with pytest.raises(ValueError):
            slice_unpacked_cols(w, e, m, 32, 128)


def _row_rank_main(rank, world, port, oc, ic, batch, mode, result_dir):
    import torch.distributed as dist
    import oracle
    from fp6_llm_b200.formats import random_codes_layer
    from fp6_llm_b200.sharding import plan_cols, reduce_partials, slice_unpacked_cols
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w, s = random_codes_layer(oc, ic, 3, 2, seed=13, scale_lo=0.01, scale_hi=0.1)
        x = torch.randn(batch, ic, generator=torch.Generator().manual_seed(6)).half()
        k0, k1 = plan_cols(ic, world)[rank]
        wk = slice_unpacked_cols(w, 3, 2, k0, k1)
        # the rank's GEMM is played by the oracle; fp32 partials keep the comparison exact up to the summation order
        local = torch.from_numpy(oracle.linear(x[:, k0:k1].contiguous().numpy(), wk.numpy(), s.numpy())).float()
        out = reduce_partials(local, mode)
        torch.save(out, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["all_reduce", "reduce_scatter"])
def test_two_rank_row_parallel_matches_unsharded(oracle_mod, tmp_path, mode):
    from fp6_llm_b200.formats import random_codes_layer
    oc, ic, batch, world = 512, 192, 5, 2          # 3 column units over 2 ranks: 128 + 64
    mp.spawn(_row_rank_main, args=(world, _free_port(), oc, ic, batch, mode, str(tmp_path)), nprocs=world, join=True)
    w, s = random_codes_layer(oc, ic, 3, 2, seed=13, scale_lo=0.01, scale_hi=0.1)
    x = torch.randn(batch, ic, generator=torch.Generator().manual_seed(6)).half()
    expect = torch.from_numpy(oracle_mod.linear(x.numpy(), w.numpy(), s.numpy())).float()
    for r in range(world):
        got = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        want = expect if mode == "all_reduce" else expect[:, r * oc // world:(r + 1) * oc // world]
        assert got.shape == want.shape
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-5 * float(expect.abs().max()))
