"""Memory-safety and repeatability checks that stand in for a sanitizer run: output buffers with guard words
either side, the same call twice, and a state dict saved and restored in the middle of a run."""
import io
import logging

import pytest
import torch

pytestmark = pytest.mark.gpu
LOG = logging.getLogger("test")
GUARD = 4096          # elements of guard either side


@pytest.fixture(scope="module")
def ops():
    from moddit_b200 import ops as _ops
    return _ops


def _guarded(shape, dtype, fill):
    """A contiguous tensor of `shape` in the middle of a larger buffer filled with `fill`."""
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((n + 2 * GUARD,), fill, device="cuda", dtype=dtype)
    return buf, buf[GUARD:GUARD + n].view(*shape)


def _guards_intact(buf, fill):
    return bool((buf[:GUARD] == fill).all()) and bool((buf[-GUARD:] == fill).all())


def _inputs(H=2, grid=(4, 16, 16), D=128, text=128, seed=11):
    from moddit_b200 import synth
    return synth.make_qkv(heads=H, grid=grid, head_dim=D, text_tokens=text, seed=seed, device=torch.device("cuda"))


@pytest.mark.parametrize("N", [1152, 1100])       # the second: a ragged last tile
def test_sparse_forward_stays_inside_its_output(ops, N):
    q, k, v = [t[:, :, :N].contiguous() for t in _inputs()]
    nb = (N + 127) // 128
    mask = torch.rand(2, nb, nb, device="cuda") < 0.5
    mask |= torch.eye(nb, device="cuda", dtype=torch.bool)
    lists = ops.tile_lists(mask, 128, N)
    buf, out = _guarded(q.shape, q.dtype, 7.0)
    got = ops.sparse_attn_fwd(q, k, v, lists.counts, lists.entries, order=lists.order, out=out)
    assert got.data_ptr() == out.data_ptr() and _guards_intact(buf, 7.0)
    again = ops.sparse_attn_fwd(q, k, v, lists.counts, lists.entries, order=lists.order)
    assert torch.equal(again, out)                 # same call, same bits


def test_prologue_stays_inside_its_outputs(ops):
    H, D, S, bs = 3, 128, 333, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    proj = [torch.randn(1, S, H * D, device="cuda", generator=g).bfloat16() for _ in range(3)]
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    ang = torch.rand(S, D // 2, device="cuda", generator=g)
    bufs, outs = zip(*[_guarded((1, H, S, D), torch.bfloat16, 5.0) for _ in range(3)])
    pbufs, pools = zip(*[_guarded((1, H, (S + bs - 1) // bs, D), torch.float32, 5.0) for _ in range(2)])
    kw = dict(num_heads=H, norm="rms_head", q_weight=w, k_weight=w, rope_cos=ang.cos().contiguous(),
              rope_sin=ang.sin().contiguous(), rope_form="pair", pool_block_size=bs)
    ops.qkv_prologue(*proj, out=outs, pools=pools, **kw)
    assert all(_guards_intact(b, 5.0) for b in bufs + pbufs)
    first = [t.clone() for t in outs + pools]
    ops.qkv_prologue(*proj, out=outs, pools=pools, **kw)
    assert all(torch.equal(a, b) for a, b in zip(first, outs + pools))


def test_state_saved_and_restored_mid_run_continues_identically():
    """The per-layer state is a dict of tensors, lists and strings: torch.save / torch.load in the middle of a
    run (after the mask has been predicted) and the restored copy produce the same outputs and masks."""
    import MoD.mod.attn_mask as am
    from MoD.mod.state import create_adaptive_mask_state

    H, grid, D, bs, text = 2, (4, 16, 16), 128, 128, 128
    q, k, v = _inputs(H, grid, D, text)
    video = grid[0] * grid[1] * grid[2]

    def fresh():
        return create_adaptive_mask_state("hunyuan", H, video, text, grid[1] * grid[2], grid[0], warmup_steps=3,
                                          top_k=6, predict_T=3, block_size=bs)

    state = fresh()
    for step in range(5):
        am.SparseAttentionWithMap(q, k, v, state, LOG, current_step=step)
    buf = io.BytesIO()
    torch.save(state, buf)
    buf.seek(0)
    restored = torch.load(buf, weights_only=False)
    assert set(restored) == set(state)
    for step in range(5, 9):                      # sparse steps and a refresh step (predict_T = 3)
        a, _ = am.SparseAttentionWithMap(q, k, v, state, LOG, current_step=step)
        b, _ = am.SparseAttentionWithMap(q, k, v, restored, LOG, current_step=step)
        assert torch.equal(a, b) and torch.equal(state["mask"], restored["mask"])


def test_nvtx_ranges_can_be_switched_on(ops):
    x = torch.randn(1, 2, 256, 128, device="cuda").bfloat16()
    want = ops.pool_blocks(x, 128)
    ops.nvtx_ranges(True)
    try:
        assert torch.equal(ops.pool_blocks(x, 128), want)
    finally:
        ops.nvtx_ranges(False)


@pytest.mark.parametrize("mode", ["pooled", "replay", "radial", "spargeattn", "full", "use_dense"])
def test_an_expired_wait_is_reported_by_the_next_call_in_every_mode(ops, mode):
    """A kernel that gives up a bounded wait leaves a code in the device's status words.  No kernel is made to
    fail here: the test writes the words itself, as such a kernel would have, behind one healthy call; the next
    call of the state machine - whatever the mode - must raise, and the call after that must run again."""
    from MoD.mod.attn_mask import SparseAttentionWithMap
    from MoD.mod.state import create_adaptive_mask_state
    from moddit_b200._lib import ModditError
    q, k, v = _inputs(H=2, grid=(4, 16, 16), D=128, text=0, seed=13)
    video = q.shape[2]
    sparse_type = mode if mode in ("radial", "spargeattn", "full") else "mod-dit"
    state = create_adaptive_mask_state("wan", 2, video, 0, 256, 4, warmup_steps=2, top_k=4, predict_T=3, block_size=128,
                                       sparse_type=sparse_type)
    if mode == "pooled":
        state["score_producer"] = "pooled"
    kw = dict(use_dense=True) if mode == "use_dense" else {}
    dev = q.device
    ops.check_health(dev)
    for step in range(3):                                   # healthy calls: priming steps and one later step
        SparseAttentionWithMap(q, k, v, state, LOG, current_step=step, **kw)
    torch.cuda.synchronize(dev)
    ops.check_posted_status(dev)                            # nothing to report
    ops._status_words(dev).copy_(torch.tensor([3, 17, 1, 5], dtype=torch.int32))
    SparseAttentionWithMap(q, k, v, state, LOG, current_step=3, **kw)     # its launch posts the words
    torch.cuda.synchronize(dev)
    with pytest.raises(ModditError, match="bounded wait expired.*code=3 block=17 role=1 position=5"):
        SparseAttentionWithMap(q, k, v, state, LOG, current_step=4, **kw)
    assert ops._status_words(dev).tolist() == [0, 0, 0, 0]  # cleared: the caller may carry on
    SparseAttentionWithMap(q, k, v, state, LOG, current_step=4, **kw)
    torch.cuda.synchronize(dev)
    ops.check_health(dev)


def test_all_true_stand_in_mask_uses_exactly_the_valid_keys(ops):
    """A mask of another shape stands for "keep everything" (the dense steps pass one): like the reference's dense
    branch (MoD/mod/attn_mask.py:268-276) every row then sees exactly the valid keys, not the 64-rounded border."""
    from MoD.mod.attn_mask import AttentionSparseEngine
    from oracle import moddit_oracle as orc
    g = torch.Generator(device="cuda").manual_seed(17)       # plain noise: every key matters to every query
    q, k, v = (torch.randn(1, 2, 640, 128, device="cuda", generator=g).bfloat16() for _ in range(3))
    S, video = q.shape[2], 512
    valid = video + 37                                      # not a multiple of 64
    pdm = (torch.arange(S, device="cuda") < valid).unsqueeze(0).expand(S, S).contiguous()
    stand_in = torch.ones(2, 4, 4, device="cuda", dtype=torch.bool)       # video-region shape, not the sequence's
    out = AttentionSparseEngine(q, k, v, stand_in, pre_defined_mask=pdm, video_token_num=video, block_size=128)
    nb = S // 128
    ref = orc.masked_attention(q.cpu(), k.cpu(), v.cpu(), torch.ones(1, nb, nb, dtype=torch.bool), 128,
                               q_split=video, kv_len_lo=valid, kv_len_hi=valid)
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
    rounded = orc.masked_attention(q.cpu(), k.cpu(), v.cpu(), torch.ones(1, nb, nb, dtype=torch.bool), 128,
                                   q_split=video, kv_len_lo=(valid + 63) // 64 * 64, kv_len_hi=valid)
    assert (ref - rounded).abs().max().item() > 1e-3        # the two rules do differ on this input
    assert (out.float().cpu() - ref).abs().max().item() < (out.float().cpu() - rounded).abs().max().item()
