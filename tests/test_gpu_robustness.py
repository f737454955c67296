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
