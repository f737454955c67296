"""GPU checks of the `--sparse_type spargeattn` comparison mode built from this library's kernels: the block
self-similarity and top-k block selection against the oracle, and the whole call against masked attention."""
import logging
import math

import pytest
import torch

from oracle import moddit_oracle as orc

pytestmark = pytest.mark.gpu
LOG = logging.getLogger("test")


@pytest.fixture(scope="module")
def ops():
    from moddit_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,bs,N", [(128, 128, 640), (64, 64, 448), (128, 64, 200), (64, 128, 385)])
def test_block_similarity(ops, dtype, D, bs, N):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, 3, N, D, generator=g)
    x[:, 0] = x[:, 0, :1] + 0.05 * x[:, 0]            # head 0: nearly parallel rows, similarity near 1
    x[:, 1, 5] = 0                                     # a zero row contributes nothing
    x = x.to(dtype)
    center = torch.randn(1, 3, D, generator=g) * 0.3
    for c in (None, center):
        ref = orc.block_similarity(x, bs, c)
        got = ops.block_similarity(x.cuda(), bs, None if c is None else c.cuda()).cpu()
        assert got.shape == ref.shape
        assert torch.allclose(got, ref, rtol=1e-4, atol=1e-6)
    assert ops.block_similarity(x.cuda(), bs)[0, 0].min().item() > 0.9


@pytest.mark.parametrize("n,count", [(7, 3), (64, 32), (130, 65), (300, 1), (33, 33)])
def test_select_topk_blocks(ops, n, count):
    g = torch.Generator().manual_seed(n)
    dark = torch.rand(2, n, n, generator=g).half()
    dark[0, :, : n // 2] = dark[0, :, : n // 2].round()          # many ties: the lowest index wins
    rf = torch.rand(2, n, generator=g) < 0.1
    ck = torch.rand(2, n, generator=g) < 0.1
    for row_full, col_keep in ((None, None), (rf, None), (rf, ck)):
        ref = orc.select_topk_blocks(dark, count, row_full, col_keep)
        got = ops.select_topk_blocks(dark.cuda(), count, None if row_full is None else row_full.cuda(),
                                     None if col_keep is None else col_keep.cuda()).cpu()
        assert torch.equal(got, ref)
    assert int(ops.select_topk_blocks(dark.cuda(), count).sum()) == 2 * n * count


@pytest.mark.parametrize("model_type,threshold", [("hunyuan", 0.0), ("wan", 0.3)])
def test_spargeattn_step(ops, model_type, threshold):
    import MoD.mod.attn_mask as am
    from MoD.mod.state import create_adaptive_mask_state
    from moddit_b200 import synth

    H, grid, D, bs = 2, (4, 16, 16), 128, 128
    text = 128 if model_type == "hunyuan" else 0
    q, k, v = synth.make_qkv(heads=H, grid=grid, head_dim=D, text_tokens=text, seed=9, device=torch.device("cuda"))
    video = grid[0] * grid[1] * grid[2]
    N = video + text
    nb = N // bs
    state = create_adaptive_mask_state(model_type, H, video, text, grid[1] * grid[2], grid[0], block_size=bs,
                                       sparse_type="spargeattn")
    state["spargeattn_sim_threshold"] = threshold
    out, info = am.SparseAttentionWithMap(q, k, v, state, LOG, current_step=7)
    assert info == {"mode": "warmup", "mask": None}
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    dark = orc.pooled_darkness_map(orc.pool_blocks(qc, bs), orc.pool_blocks(kc, bs), q_block_offset=0,
                                   k_block_offset=0, video_blocks=nb, scale=D ** -0.5)[0]
    gpu_dark = ops.pooled_map(ops.pool_blocks(q, bs), ops.pool_blocks(k, bs), q_block_offset=0, k_block_offset=0,
                              video_blocks=nb, scale=D ** -0.5)[0].cpu()
    assert (gpu_dark.float() - dark.float()).abs().max().item() <= 2e-3
    row_full = col_keep = None
    if threshold > 0:
        kbar = ops.pool_blocks(k, bs)                                  # the step's own mean key: same operations
        rows = torch.full((nb,), float(bs), device="cuda")
        centre = ((kbar * rows[None, None, :, None]).sum(dim=2) / float(N)).contiguous()
        assert torch.allclose(centre.cpu(), kc.float().mean(dim=2), atol=1e-5)
        q_sim, k_sim = ops.block_similarity(q, bs), ops.block_similarity(k, bs, centre)
        assert torch.allclose(q_sim.cpu(), orc.block_similarity(qc, bs), rtol=1e-3, atol=1e-5)
        assert torch.allclose(k_sim.cpu(), orc.block_similarity(kc, bs, centre.cpu()), rtol=1e-3, atol=1e-5)
        row_full, col_keep = q_sim[0].cpu() < threshold, k_sim[0].cpu() < threshold
    mask = orc.select_topk_blocks(gpu_dark, math.ceil(0.5 * nb), row_full, col_keep)
    assert torch.equal(state["mask"].cpu(), mask)
    if threshold == 0:
        assert abs(mask.float().mean().item() - math.ceil(0.5 * nb) / nb) < 1e-6
    ref = orc.masked_attention(qc, kc, vc, state["mask"].cpu(), bs)
    err = (out.float().cpu() - ref).abs().max().item()
    rel = ((out.float().cpu() - ref).norm() / ref.norm()).item()
    assert err <= 2e-2 and rel <= 1e-2
