"""One rank of the two-GPU test of the fused exchange (started by tests/test_gpu_gather.py through torch.distributed.run).

Every rank builds the whole seeded layer, keeps its own shard, runs the sharded layer through PeerExchange several
times (all rotating buffers, several shapes) and checks the full [B, OC] result it ends up with against the
shards computed locally with the plain entry point (identical bits: same kernel, same plan per shard).  A second
part runs same-shape layers back to back without any host synchronisation and looks at result k only after call k+1
has been issued, which is the lifetime PeerExchange documents."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import random_codes_layer
    from fp6_llm_b200.sharding import PeerExchange, ShardedFPxLinear, plan_rows

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    exchange = PeerExchange()
    for oc, ic, batches, seed in ((4096, 4096, (1, 8, 8, 33), 1), (2560, 1024, (5, 5, 5, 140), 2)):
        w, s = random_codes_layer(oc, ic, 3, 2, seed, scale_lo=0.01, scale_hi=0.1)
        w, s = w.to(dev), s.to(dev)
        plan = plan_rows(oc, world)
        packed = [f.weight_prepacking_cpu(w[a:b].contiguous()) for a, b in plan]
        scales = [s[a:b].contiguous() for a, b in plan]
        layer = ShardedFPxLinear(packed[rank], scales[rank], plan, rank, 3, 2, exchange=exchange)
        for i, bs in enumerate(batches):
            x = torch.randn(bs, ic, generator=torch.Generator().manual_seed(100 * seed + i)).half().to(dev)
            got = layer.forward(x, 0)
            assert f.device_status() == 0, "a wait inside a kernel gave up"
            for r, (a, b) in enumerate(plan):
                expect = f.linear_forward_cuda(x, packed[r], scales[r], 0)
                assert torch.equal(got[:, a:b], expect), f"rank {rank}: rows of rank {r} differ (OC={oc}, B={bs}, call {i})"
    # back to back: no host synchronisation between the calls; result k is copied out only after call k+1 was issued
    oc, ic, bs = 2048, 2048, 16
    w, s = random_codes_layer(oc, ic, 3, 2, 9, scale_lo=0.01, scale_hi=0.1)
    w, s = w.to(dev), s.to(dev)
    plan = plan_rows(oc, world)
    packed = [f.weight_prepacking_cpu(w[a:b].contiguous()) for a, b in plan]
    scales = [s[a:b].contiguous() for a, b in plan]
    layer = ShardedFPxLinear(packed[rank], scales[rank], plan, rank, 3, 2, exchange=exchange)
    xs = [torch.randn(bs, ic, generator=torch.Generator().manual_seed(900 + i)).half().to(dev) for i in range(7)]
    kept, previous = [], None
    for x in xs:
        got = layer.forward(x, 0)
        if previous is not None:
            kept.append(previous.clone())     # in stream order: after call k+1 was issued, before call k+2
        previous = got
    kept.append(previous.clone())
    torch.cuda.synchronize(dev)
    assert f.device_status() == 0, "a wait inside a kernel gave up"
    for i, x in enumerate(xs):
        expect = torch.cat([f.linear_forward_cuda(x, packed[r], scales[r], 0) for r in range(world)], dim=1)
        assert torch.equal(kept[i], expect), f"rank {rank}: back-to-back call {i} differs"
    # orderly exit: everything done on every rank, buffers and mappings dropped, then the process group
    torch.cuda.synchronize(dev)
    dist.barrier()
    exchange.close()
    dist.barrier()
    if rank == 0:
        print("gather worker ok", flush=True)
    sys.stdout.flush()
    import threading
    watchdog = threading.Timer(30.0, lambda: os._exit(0))   # only if the communicator's teardown does not return
    watchdog.daemon = True
    watchdog.start()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
