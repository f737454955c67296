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

# Pooling on the sequence shards (halo rows + means sent to the head owners) against pooling the gathered
# heads: bit-exact, with a shard boundary inside a block and a short last block; then one full step of the
# state machine fed with those means while query and key arrive on a side stream.
CHILD_POOL = r'''
import os, sys, logging, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "mod-dit_b200"))
from moddit_b200 import dist as md, ops
from MoD.mod.attn_mask import SparseAttentionWithMap
from MoD.mod.state import create_adaptive_mask_state
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
for (H, N, D, bs, dt) in ((4, 1344, 128, 128, torch.bfloat16), (2, 1472, 64, 64, torch.float16)):
    g = torch.Generator().manual_seed(11)
    q, k = (torch.randn(1, H, N, D, generator=g).to(dt) for _ in range(2))
    b, e = md.shard_bounds(N, world, rank)
    hb, he = md.shard_bounds(H, world, rank)
    pr = md.PeerResharder(H, N, D, dt, dev, n_inputs=2)
    pr.enable_pooling(bs)
    assert pr.pool_part[2] + pr.pool_part[3] > 0          # a boundary really cuts a block
    qs, ks = q[:, :, b:e].contiguous().to(dev), k[:, :, b:e].contiguous().to(dev)
    for _ in range(2):                                    # buffers are reused across calls
        qbar, kbar = pr.pool_to_head(qs, ks)
        assert torch.equal(qbar, ops.pool_blocks(q[:, hb:he].contiguous().to(dev), bs))
        assert torch.equal(kbar, ops.pool_blocks(k[:, hb:he].contiguous().to(dev), bs))
    del pr

# state machine: the step fed with shard-pooled means equals the step that pools the gathered heads
H, T, F, D, bs = 4, 5, 256, 128, 128
N = T * F + 128                                           # 1408: 704 rows per rank, boundary inside block 5
g = torch.Generator().manual_seed(3)
q, k, v = (torch.randn(1, H, N, D, generator=g).bfloat16() for _ in range(3))
b, e = md.shard_bounds(N, world, rank)
hb, he = md.shard_bounds(H, world, rank)
pr = md.PeerResharder(H, N, D, torch.bfloat16, dev)
pr.enable_pooling(bs)
log = logging.getLogger("t")
def state():
    st = create_adaptive_mask_state("hunyuan", he - hb, T * F, 128, F, T, warmup_steps=2, top_k=6, predict_T=5, block_size=bs)
    st["score_producer"] = "pooled"
    return st
st_a, st_b, st_c = state(), state(), state()
side = torch.cuda.Stream(device=dev)
for step in range(4):
    qh, kh, vh = (t[:, hb:he].contiguous().to(dev) for t in (q, k, v))
    out_a, _ = SparseAttentionWithMap(qh, kh, vh, st_a, log, current_step=step)
    shard = [t[:, :, b:e].contiguous().to(dev) for t in (q, k, v)]
    main = torch.cuda.current_stream(dev)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        # after the first step the previous use of the buffers ended with a closing barrier (finish_output below):
        # the opening barriers may be skipped
        qs, ks = pr.seq_to_head_many(shard[:2], [0, 1], channel=0, quiesced=step > 0)
        vs = pr.seq_to_head(shard[2], 2, channel=0, quiesced=step > 0)
        ready = torch.cuda.Event(); ready.record(side)
    pooled = pr.pool_to_head(shard[0], shard[1], channel=1, quiesced=step > 0)
    out_b, _ = SparseAttentionWithMap(qs, ks, vs, st_b, log, current_step=step, value_ready=ready, qk_ready=ready,
                                      pooled_qk=pooled)
    assert torch.equal(out_a, out_b), step
    if step == 2:
        assert torch.equal(st_a["mask"], st_b["mask"])
    # (c) the heads arrive in two groups and the sparse forward runs once per group, scattering its rows to the peers
    side.wait_stream(main)
    with torch.cuda.stream(side):
        (qg, kg, vg), group_ready = pr.seq_to_head_groups(shard, [0, 1, 2], 2, channel=0)
    pooled = pr.pool_to_head(shard[0], shard[1], channel=1)
    st_c["_head_groups"] = 2
    scatter = pr.begin_output(channel=1)
    out_c, _ = SparseAttentionWithMap(qg, kg, vg, st_c, log, current_step=step, pooled_qk=pooled,
                                      head_group_ready=group_ready, output_scatter=scatter)
    out_c = pr.finish_output(channel=1).clone() if out_c is None else pr.head_to_seq(out_c, channel=1).clone()
    gathered = [torch.empty_like(out_a) for _ in range(world)]
    dist.all_gather(gathered, out_a.contiguous())
    assert torch.equal(out_c, torch.cat(gathered, dim=1)[:, :, b:e]), step
    torch.cuda.synchronize(); dist.barrier()
ops.raise_on_status(dev)
dist.barrier(); dist.destroy_process_group()
print("CHILD_OK", rank)
'''


def _run_two_ranks(tmp_path, text):
    script = tmp_path / "child.py"
    script.write_text(text)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), str(script), ROOT]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    first = res.stderr.find("Traceback")            # the child's own traceback comes before the launcher's summary
    assert res.returncode == 0, res.stdout[-1000:] + res.stderr[max(first, 0):][:3000]
    assert res.stdout.count("CHILD_OK") == 2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_shard_pooling_matches_gathered_pooling_two_gpus(tmp_path):
    _run_two_ranks(tmp_path, CHILD_POOL)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_reshard_and_fused_scatter_two_gpus(tmp_path):
    _run_two_ranks(tmp_path, CHILD)
