"""Head sharding across ranks (the only multi-GPU structure of the path), run as 2 gloo ranks on CPU."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    import bench
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = bench.WORKLOADS["cfg4"]
        lo, hi, qlo, qhi = bench.shard_heads(w["hq"], w["hkv"], rank, world)
        lens = bench.make_lengths(w["lens"], w["batch"], seed=1234)
        bt = bench.make_block_tables((lens + 15) // 16)
        # every rank derives the same lengths and block tables from the seed (they are replicated, not exchanged)
        ref_lens, ref_bt = lens.clone(), bt.clone()
        dist.broadcast(ref_lens, 0)
        dist.broadcast(ref_bt, 0)
        same = bool(torch.equal(ref_lens, lens) and torch.equal(ref_bt, bt))
        # head ranges partition the heads
        mine = torch.tensor([lo, hi, qlo, qhi])
        allr = [torch.zeros(4, dtype=torch.long) for _ in range(world)]
        dist.all_gather(allr, mine)
        # the step time of the job is the slowest rank's
        t = torch.tensor([10.0 + rank])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        q.put((rank, same, [a.tolist() for a in allr], float(t)))
    finally:
        dist.destroy_process_group()


def test_head_sharding_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 500
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, same, ranges, tmax in res:
        assert same
        assert ranges == [[0, 4, 0, 32], [4, 8, 32, 64]]
        assert tmax == 11.0


def test_shard_heads_covers_all_world_sizes():
    sys.path.insert(0, ROOT)
    import bench
    for world in (1, 2, 4, 8):
        kv, qh = [], []
        for r in range(world):
            lo, hi, qlo, qhi = bench.shard_heads(64, 8, r, world)
            kv += list(range(lo, hi))
            qh += list(range(qlo, qhi))
            assert all(h // 8 in range(lo, hi) for h in range(qlo, qhi))      # a query head stays with its KV head
        assert kv == list(range(8)) and qh == list(range(64))
    lens = bench.make_lengths("lognormal:4096:1.0:128:65536", 256, seed=1)
    assert lens.min() >= 128 and lens.max() <= 65536
    bt = bench.make_block_tables((lens + 15) // 16)
    used = torch.cat([bt[s, :int((lens[s] + 15) // 16)] for s in range(256)])
    assert used.unique().numel() == used.numel() == int(((lens + 15) // 16).sum())
