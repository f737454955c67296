"""Two-GPU test of the peer-memory re-shard and of the attention kernel's fused output scatter.

Runs as child processes (one per GPU) and is skipped on boxes with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "mod-dit_b200"))
from moddit_b200 import dist as md, ops
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
H, N, D, bs = 4, 2048, 128, 128
g = torch.Generator().manual_seed(5)
q, k, v = (torch.randn(1, H, N, D, generator=g).bfloat16() for _ in range(3))
mask = torch.rand(H, N // bs, N // bs, generator=g) < 0.4
mask[:, torch.arange(N // bs), torch.arange(N // bs)] = True
b, e = md.shard_bounds(N, world, rank)
hb, he = md.shard_bounds(H, world, rank)
pr = md.PeerResharder(H, N, D, torch.bfloat16, dev)
qs, ks = pr.seq_to_head_many([q[:, :, b:e].contiguous().to(dev), k[:, :, b:e].contiguous().to(dev)], [0, 1])
vs = pr.seq_to_head(v[:, :, b:e].contiguous().to(dev), 2)
assert torch.equal(qs.cpu(), q[:, hb:he]) and torch.equal(ks.cpu(), k[:, hb:he]) and torch.equal(vs.cpu(), v[:, hb:he])
assert torch.equal(md.seq_to_head(q[:, :, b:e].contiguous().to(dev)).cpu(), q[:, hb:he])      # NCCL path agrees
lists = ops.tile_lists(mask[hb:he].to(dev), bs, N)
ref = ops.sparse_attn_fwd(qs, ks, vs, lists.counts, lists.entries, order=lists.order)
# (a) copy-based output exchange, (b) scatter fused into the kernel epilogue: both must equal the local result
out_a = pr.head_to_seq(ref).clone()
scatter = pr.begin_output()
ops.sparse_attn_fwd(qs, ks, vs, lists.counts, lists.entries, order=lists.order, scatter=scatter)
out_b = pr.finish_output().clone()
gathered = [torch.empty_like(ref) for _ in range(world)]
dist.all_gather(gathered, ref)
full = torch.cat(gathered, dim=1)                      # (1, H, N, D) from every rank's heads
assert torch.equal(out_a, full[:, :, b:e]) and torch.equal(out_b, full[:, :, b:e])
ops.raise_on_status(dev)
dist.barrier(); dist.destroy_process_group()
print("CHILD_OK", rank)
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_reshard_and_fused_scatter_two_gpus(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), str(script), ROOT]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("CHILD_OK") == 2
