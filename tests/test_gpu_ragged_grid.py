"""Sequences the reference refuses (MoD/mod/attn_mask.py:165, MoD/mod/triton_flash_sparsity.py:157-160): video and
text regions that are not whole numbers of blocks.  The mean-pooled producer accepts them on the block grid
`block_geometry` defines (a short last block; a block holding any text token is a text block).  Small shapes,
every stage against the CPU oracle; the oracle of the output is fp32 attention under the token-expanded mask."""
import logging

import pytest
import torch

from oracle import moddit_oracle as orc

pytestmark = pytest.mark.gpu
LOG = logging.getLogger("ragged")


@pytest.mark.parametrize("model_type,bs,D,grid,text", [
    ("cogvideox", 64, 64, (4, 12, 17), 40),      # 816 video + 40 text: 14 blocks, 1 text block, 13 video blocks
    ("hunyuan", 128, 128, (3, 10, 19), 100),     # 570 video + 100 text: 6 blocks, 4 video blocks
    ("wan", 64, 64, (5, 9, 11), 0),              # 495 tokens: 8 blocks, the last holds 47
])
@pytest.mark.parametrize("selector", ["topk_lines", "cumulative_mass"])
def test_ragged_shapes_through_the_state_machine(model_type, bs, D, grid, text, selector):
    from MoD.mod.attn_mask import SparseAttentionWithMap
    from MoD.mod.state import create_adaptive_mask_state
    from moddit_b200 import ops, synth
    H = 2
    T, Hh, Ww = grid
    video = T * Hh * Ww
    N = video + text
    q, k, v = synth.make_qkv(heads=H, grid=grid, head_dim=D, text_tokens=text, text_first=model_type == "cogvideox",
                             seed=21, device="cuda")
    nb, n, off = orc.block_geometry(model_type, bs, video, text, N)
    assert N % bs != 0 or video % bs != 0
    bpf = max(1, (Hh * Ww) // bs)
    top_k = 5
    state = create_adaptive_mask_state(model_type, H, video, text, Hh * Ww, T, warmup_steps=2, top_k=top_k, predict_T=4,
                                       block_size=bs)
    state["blocks_per_frame"] = bpf
    state["score_producer"] = "pooled"
    state["selector"] = selector
    state["mass_threshold"] = 0.9
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    dark_ref = orc.pooled_darkness_map(orc.pool_blocks(qc, bs), orc.pool_blocks(kc, bs), q_block_offset=off,
                                       k_block_offset=off, video_blocks=n, scale=D ** -0.5)[0]
    for step in range(3):
        out, info = SparseAttentionWithMap(q, k, v, state, LOG, current_step=step)
        assert out.shape == q.shape
        dark = state["prev_full_maps"].cpu()
        assert dark.shape == (H, n, n)
        assert (dark.float() - dark_ref.float()).abs().max().item() <= 2e-3
        if step == 0:
            ref = orc.masked_attention(qc, kc, vc, torch.ones(1, nb, nb, dtype=torch.bool), bs)
        else:
            if selector == "cumulative_mass":
                vm = orc.select_mass(dark, 0.9)
                if model_type == "wan":
                    want = vm
                else:
                    want = torch.ones(H, nb, nb, dtype=torch.bool)
                    want[:, off:off + n, off:off + n] = vm
            else:
                gh = [{k_: v_.cpu() for k_, v_ in f_.items()} for f_ in state["features_history"][-2:]]
                f = orc.solve_features(orc.compute_mts(dark, bpf), n, bpf, 1.0)
                for k_ in ("c", "d", "b_d"):
                    assert torch.allclose(gh[-1][k_], f[k_].float(), atol=5e-4, rtol=1e-3)
                lines = orc.choose_topk_lines(gh[0], gh[1], top_k, 4)
                want = orc.generate_mask_from_lines(model_type=model_type, block_size=bs, video_token_num=video,
                                                    text_token_num=text, seq_len=N, blocks_per_frame=bpf,
                                                    selected_lines=lines, mode=orc.check_bd_values(gh[1]["b_d"], 1.0))
            assert state["mask"].shape == (H, nb, nb)
            assert torch.equal(state["mask"].cpu(), want)
            ref = orc.masked_attention(qc, kc, vc, want, bs)
        got = out.float().cpu()
        assert torch.isfinite(got).all()
        assert (got - ref).abs().max().item() <= 2e-2
        assert ((got - ref).norm() / ref.norm()).item() <= 1e-2
    ops.check_health(q.device)


def test_replay_producer_still_refuses_unaligned_video_like_the_reference():
    from MoD.mod.triton_flash_sparsity import flash_attn_with_sparsity_map
    q = torch.randn(1, 2, 856, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="divisible"):
        flash_attn_with_sparsity_map(q, q, q, threshold=1e-3, block_size=64, model_type="cogvideox",
                                     video_token_num=816, text_token_num=40)
