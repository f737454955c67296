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


def _load_dist_module():
    import importlib.util
    spec = importlib.util.spec_from_file_location("moddit_dist_plain",
                                                  os.path.join(ROOT, "mod-dit_b200", "moddit_b200", "dist.py"))
    md = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(md)
    return md


def test_pool_partition_covers_every_block_once():
    """Shard-side pooling: every block has exactly one producer, halos and tails of neighbours agree, and
    block means taken from (halo ++ own rows) equal the means of the whole sequence."""
    md = _load_dist_module()
    for N, bs, world in ((115456, 128, 8), (115456, 128, 4), (115456, 128, 2), (1344, 128, 2), (75600, 64, 8),
                         (1472, 64, 2), (1024, 128, 8)):
        parts = [md.pool_partition(N, bs, world, r) for r in range(world)]
        nb = (N + bs - 1) // bs
        assert parts[0][0] == 0 and parts[0][2] == 0 and parts[-1][1] == nb and parts[-1][3] == 0
        for a, b in zip(parts, parts[1:]):
            assert a[1] == b[0] and a[3] == b[2] and 0 <= a[3] < bs
        if N > 20000:
            continue
        ns = N // world
        x = torch.arange(N, dtype=torch.float64) ** 2
        want = torch.stack([x[i * bs:(i + 1) * bs].mean() for i in range(nb)])
        got = torch.empty(nb, dtype=torch.float64)
        for r, (first, end, halo, tail) in enumerate(parts):
            rows = torch.cat([x[r * ns - halo:r * ns], x[r * ns:(r + 1) * ns]])
            for i in range(end - first):
                got[first + i] = rows[i * bs:(i + 1) * bs].mean()
        assert torch.equal(got, want)
    import pytest
    with pytest.raises(ValueError):
        md.pool_partition(1000, 128, 8, 0)      # a shard shorter than a block
    with pytest.raises(ValueError):
        md.pool_partition(1001, 128, 2, 0)


def test_group_pieces_place_every_row_once():
    """The exchange by groups of heads, emulated on byte arrays for 2, 4 and 8 ranks: after every rank's pieces of
    groups 0..g have been copied, the owners hold exactly the heads of those groups, and after the last group the
    whole head-major tensor; nothing is written twice."""
    import numpy as np
    md = _load_dist_module()
    for world, H, N, D, groups in ((2, 8, 12, 2, 3), (4, 24, 16, 2, 2), (8, 24, 32, 1, 3), (8, 24, 32, 1, 1), (4, 8, 8, 3, 5)):
        hp, ns, esize, T = H // world, N // world, 2, 3
        row, head = ns * D * esize, N * D * esize
        full = [np.random.default_rng(t).integers(1, 255, size=(H, N, D * esize), dtype=np.uint8) for t in range(T)]
        # one flat address space: shards of every rank, then owners' buffers
        shard_bytes, buf_bytes = H * row, hp * head
        x_ptr = lambda r, t: (r * T + t) * shard_bytes
        b_ptr = lambda r, t: world * T * shard_bytes + (r * T + t) * buf_bytes
        mem = np.zeros(world * T * (shard_bytes + buf_bytes), dtype=np.uint8)
        written = np.zeros_like(mem)
        for r in range(world):
            for t in range(T):
                mem[x_ptr(r, t):x_ptr(r, t) + shard_bytes] = full[t][:, r * ns:(r + 1) * ns].reshape(-1)
        plans = [md.group_pieces(world, r, hp, groups, row, head, [x_ptr(r, t) for t in range(T)],
                                 [[b_ptr(p, t) for p in range(world)] for t in range(T)]) for r in range(world)]
        n_groups = len(plans[0])
        assert all(len(p) == n_groups for p in plans) and n_groups == min(groups, hp, -(-hp // -(-hp // min(groups, hp))))
        hpg = -(-hp // min(groups, hp))
        for g in range(n_groups):
            for r in range(world):
                src, dst, rows = plans[r][g]
                assert len(src) == len(dst) == world * T
                for s_, d_ in zip(src, dst):
                    for j in range(rows):
                        mem[d_ + j * head:d_ + j * head + row] = mem[s_ + j * row:s_ + j * row + row]
                        written[d_ + j * head:d_ + j * head + row] += 1
            upto = min(hp, (g + 1) * hpg)
            for r in range(world):
                for t in range(T):
                    got = mem[b_ptr(r, t):b_ptr(r, t) + buf_bytes].reshape(hp, N, D * esize)
                    assert np.array_equal(got[:upto], full[t][r * hp:r * hp + upto])
        assert written[world * T * shard_bytes:].min() == 1 and written.max() == 1

