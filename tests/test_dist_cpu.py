"""World-size-2 gloo test of the sequence<->head re-shard index math (CPU only)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, os.path.join(ROOT, "mod-dit_b200"))
    import importlib.util
    spec = importlib.util.spec_from_file_location("moddit_dist", os.path.join(ROOT, "mod-dit_b200", "moddit_b200", "dist.py"))
    md = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(md)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, N, D = 4, 12, 3
    full = torch.arange(H * N * D, dtype=torch.float32).reshape(1, H, N, D)
    b, e = md.shard_bounds(N, world, rank)
    mine = full[:, :, b:e].contiguous()
    heads = md.seq_to_head(mine)
    hb, he = md.shard_bounds(H, world, rank)
    ok1 = torch.equal(heads, full[:, hb:he])
    back = md.head_to_seq(heads * 2)
    ok2 = torch.equal(back, mine * 2)
    ret[rank] = bool(ok1 and ok2)
    dist.destroy_process_group()


def test_reshard_round_trip_two_ranks():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret[0] and ret[1]
