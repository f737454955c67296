"""The benchmark specification's first configuration as a parity case: B=1, 2 heads x 64, block 64, 4096 tokens
on a 4 x 32 x 32 latent grid (64 blocks, 16 per frame), seeded locality inputs, once through the reference's
line-selection path and once through the pooled producer with the cumulative-mass rule (threshold 0.9)."""
import logging

import pytest
import torch

from oracle import moddit_oracle as orc

pytestmark = pytest.mark.gpu
LOG = logging.getLogger("test")
H, GRID, D, BS = 2, (4, 32, 32), 64, 64
N = GRID[0] * GRID[1] * GRID[2]
NB, BPF = N // BS, GRID[1] * GRID[2] // BS


@pytest.fixture(scope="module")
def qkv():
    from moddit_b200 import synth
    return synth.make_qkv(heads=H, grid=GRID, head_dim=D, text_tokens=0, seed=0, device=torch.device("cuda"))


def _close(out, ref):
    diff = out.float().cpu() - ref
    assert diff.abs().max().item() <= 2e-2 and (diff.norm() / ref.norm()).item() <= 1e-2


def test_config0_reference_line_selection(qkv):
    import MoD.mod.attn_mask as am
    from MoD.mod.state import create_adaptive_mask_state
    q, k, v = qkv
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    top_k, pT, thr = 20, 5, 1e-3
    state = create_adaptive_mask_state("wan", H, N, 0, GRID[1] * GRID[2], GRID[0], warmup_steps=2, top_k=top_k,
                                       predict_T=pT, threshold=thr, block_size=BS)
    dense = orc.masked_attention(qc, kc, vc, torch.ones(1, NB, NB, dtype=torch.bool), BS)
    for step in (0, 1):
        out, _ = am.SparseAttentionWithMap(q, k, v, state, LOG, current_step=step)
        _close(out, dense)
    # the exact map against the oracle's replay of the same computation (the reference test bounds this comparison by 8.1 elements per block)
    lse, scale = orc.replay_lse(qc, kc)
    ref_map = orc.sparsity_map_replay(qc, kc, lse, softmax_scale=scale, log_threshold=torch.log(torch.tensor(thr)).item(),
                                      q_video_offset=0, k_video_offset=0, video_blocks=NB, block_size=BS)
    got_map = state["prev_full_maps"].cpu().float()
    assert ((got_map - ref_map[0].float()).abs() * BS * BS).max().item() <= 8.1
    # mask: bit-exact from the device's features, >= 99.9 % of blocks from the oracle's own fit of the device map
    hist = [{key: val.cpu() for key, val in f.items()} for f in state["features_history"][-2:]]
    modes = orc.check_bd_values(hist[1]["b_d"], 1.0)
    mask = orc.generate_mask_from_lines(model_type="wan", block_size=BS, video_token_num=N, text_token_num=0, seq_len=N,
                                        blocks_per_frame=BPF, selected_lines=orc.choose_topk_lines(hist[0], hist[1], top_k, pT),
                                        mode=modes)
    assert torch.equal(state["mask"].cpu(), mask)
    fit = orc.solve_features(orc.compute_mts(state["prev_full_maps"].cpu(), BPF), NB, BPF, 1.0)
    mask2 = orc.generate_mask_from_lines(model_type="wan", block_size=BS, video_token_num=N, text_token_num=0, seq_len=N,
                                         blocks_per_frame=BPF,
                                         selected_lines=orc.choose_topk_lines(hist[0], {x: fit[x] for x in ("c", "d", "b_d")},
                                                                              top_k, pT), mode=modes)
    assert (mask2 == mask).float().mean().item() >= 0.999
    out, _ = am.SparseAttentionWithMap(q, k, v, state, LOG, current_step=2)
    _close(out, orc.masked_attention(qc, kc, vc, mask, BS))


def test_config0_pooled_scores_cumulative_mass(qkv):
    import MoD.mod.attn_mask as am
    from MoD.mod.state import create_adaptive_mask_state
    q, k, v = qkv
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    state = create_adaptive_mask_state("wan", H, N, 0, GRID[1] * GRID[2], GRID[0], warmup_steps=2, top_k=20,
                                       predict_T=5, block_size=BS)
    state["score_producer"], state["selector"], state["mass_threshold"] = "pooled", "cumulative_mass", 0.9
    for step in (0, 1):
        out, _ = am.SparseAttentionWithMap(q, k, v, state, LOG, current_step=step)
    dark = orc.pooled_darkness_map(orc.pool_blocks(qc, BS), orc.pool_blocks(kc, BS), q_block_offset=0,
                                   k_block_offset=0, video_blocks=NB, scale=D ** -0.5)[0]
    gpu_dark = state["prev_full_maps"].cpu()
    assert (gpu_dark.float() - dark.float()).abs().max().item() <= 2e-3
    mask = orc.select_mass(gpu_dark, 0.9)           # identical pooled scores -> identical mask
    assert torch.equal(state["mask"].cpu(), mask)
    assert (orc.select_mass(dark, 0.9) == mask).float().mean().item() >= 0.999
    assert bool(mask.diagonal(dim1=1, dim2=2).all()) and 0.0 < mask.float().mean().item() < 1.0
    _close(out, orc.masked_attention(qc, kc, vc, mask, BS))
