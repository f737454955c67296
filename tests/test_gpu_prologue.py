"""GPU parity of the attention prologue (normalisation + rotary embedding + head-major layout in one pass)
against the oracle's step-by-step restatement of the reference processors."""
import pytest
import torch

from oracle import moddit_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from moddit_b200 import ops as _ops
    return _ops


def _tables(rows, D, seed):
    g = torch.Generator().manual_seed(seed)
    ang = torch.rand(rows, D // 2, generator=g) * 6.28
    return ang.cos().repeat_interleave(2, 1).contiguous(), ang.sin().repeat_interleave(2, 1).contiguous()


def _proj(B, S, W, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(B, S, W, generator=g) * (1.0 + i)).to(dtype) for i in range(3)]


def _close_after_norm(got, ref, dtype):
    """The normalised value is rounded twice to the 16-bit type; the row mean is summed in another order than
    torch sums it, so a value may land on the neighbouring grid point (1 ulp = 2^-7 relative for bfloat16,
    2^-10 for float16), and the rotation mixes the two values of a pair: bound the difference by 2 ulp of the
    pair's magnitude, and require nearly all values to be identical."""
    got, ref = got.float().cpu(), ref.float()
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    pair = ref.unflatten(-1, (-1, 2)).pow(2).sum(-1, keepdim=True).sqrt().expand(*ref.shape[:-1], -1, 2).flatten(-2)
    assert bool(((got - ref).abs() <= 2 * ulp * pair + 1e-7).all())
    assert (got == ref).float().mean().item() > 0.97


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("form", ["elementwise", "even_cos_odd_sin", "pair"])
@pytest.mark.parametrize("H,D,S,lo,hi", [(3, 128, 300, 0, 300), (2, 64, 197, 40, 197), (2, 128, 130, 0, 100)])
def test_rotary_and_layout_are_bit_exact(ops, dtype, form, H, D, S, lo, hi):
    q, k, v = _proj(2, S, H * D, dtype, 1)
    cos, sin = _tables(hi - lo, D, 2)
    if form == "elementwise":     # tables whose even and odd entries differ tell the two forms apart
        cos, sin = cos * torch.linspace(0.9, 1.1, D), sin * torch.linspace(1.1, 0.9, D)
    if form == "pair":
        cos, sin = cos[:, 0::2].contiguous(), sin[:, 0::2].contiguous()
    ref = orc.qkv_prologue(q, k, v, num_heads=H, rope_cos=cos, rope_sin=sin, rope_form=form, rope_range=(lo, hi))
    (gq, gk, gv), pools = ops.qkv_prologue(q.cuda(), k.cuda(), v.cuda(), num_heads=H, rope_cos=cos.cuda(),
                                           rope_sin=sin.cuda(), rope_form=form, rope_range=(lo, hi))
    assert pools is None
    for got, want in zip((gq, gk, gv), ref):
        assert got.shape == want.shape and got.dtype == want.dtype
        assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_hunyuan_single_stream(ops, dtype):
    """RMSNorm per head, rotary on the latent tokens, text tokens at the end untouched by the rotation; the
    projections are slices of one fused (B, S, 3*H*D) tensor; block means come out with it."""
    H, D, Sv, St, bs = 3, 128, 384, 70, 128
    S = Sv + St
    g = torch.Generator().manual_seed(5)
    fused = torch.randn(1, S, 3 * H * D, generator=g).to(dtype)
    q, k, v = fused.split(H * D, dim=2)
    qw, kw = [(1 + 0.1 * torch.randn(D, generator=g)).to(dtype) for _ in range(2)]
    cos, sin = _tables(Sv, D, 6)
    ref = orc.qkv_prologue(q, k, v, num_heads=H, norm="rms_head", q_weight=qw, k_weight=kw, rope_cos=cos,
                           rope_sin=sin, rope_range=(0, Sv))
    fd = fused.cuda()
    dq, dk, dv = fd.split(H * D, dim=2)
    (gq, gk, gv), (pq, pk) = ops.qkv_prologue(dq, dk, dv, num_heads=H, norm="rms_head", q_weight=qw.cuda(),
                                              k_weight=kw.cuda(), rope_cos=cos.cuda(), rope_sin=sin.cuda(),
                                              rope_range=(0, Sv), pool_block_size=bs)
    _close_after_norm(gq, ref[0], dtype)
    _close_after_norm(gk, ref[1], dtype)
    assert torch.equal(gv.cpu(), ref[2])
    assert torch.equal(pq, ops.pool_blocks(gq, bs)) and torch.equal(pk, ops.pool_blocks(gk, bs))


def test_hunyuan_dual_stream_appends_the_text(ops):
    """Latent and text streams are projected and normalised separately (different weights) and concatenated
    (MoD/models/hunyuan/attention_processor.py:88-106): two calls fill one buffer."""
    dtype, H, D, Sv, St, bs = torch.bfloat16, 2, 128, 256, 45, 128
    g = torch.Generator().manual_seed(7)
    vid = _proj(1, Sv, H * D, dtype, 8)
    txt = _proj(1, St, H * D, dtype, 9)
    w = [(1 + 0.1 * torch.randn(D, generator=g)).to(dtype) for _ in range(4)]
    cos, sin = _tables(Sv, D, 10)
    rv = orc.qkv_prologue(*vid, num_heads=H, norm="rms_head", q_weight=w[0], k_weight=w[1], rope_cos=cos, rope_sin=sin)
    rt = orc.qkv_prologue(*txt, num_heads=H, norm="rms_head", q_weight=w[2], k_weight=w[3])
    ref = [torch.cat([a, b], dim=2) for a, b in zip(rv, rt)]
    out, pools = ops.qkv_prologue(*[t.cuda() for t in vid], num_heads=H, norm="rms_head", q_weight=w[0].cuda(),
                                  k_weight=w[1].cuda(), rope_cos=cos.cuda(), rope_sin=sin.cuda(),
                                  total_tokens=Sv + St, pool_block_size=bs)
    out2, pools2 = ops.qkv_prologue(*[t.cuda() for t in txt], num_heads=H, norm="rms_head", q_weight=w[2].cuda(),
                                    k_weight=w[3].cuda(), out=out, dst_row0=Sv, pool_block_size=bs, pools=pools)
    assert out2[0].data_ptr() == out[0].data_ptr() and pools2[0].data_ptr() == pools[0].data_ptr()
    _close_after_norm(out[0], ref[0], dtype)
    _close_after_norm(out[1], ref[1], dtype)
    assert torch.equal(out[2].cpu(), ref[2])
    assert torch.equal(pools[0], ops.pool_blocks(out[0], bs)) and torch.equal(pools[1], ops.pool_blocks(out[1], bs))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_wan_norm_across_heads(ops, dtype):
    H, D, S = 4, 128, 333
    q, k, v = _proj(2, S, H * D, dtype, 11)
    g = torch.Generator().manual_seed(12)
    qw, kw = [(1 + 0.1 * torch.randn(H * D, generator=g)).to(dtype) for _ in range(2)]
    cos, sin = _tables(S, D, 13)
    ref = orc.qkv_prologue(q, k, v, num_heads=H, norm="rms_all_heads", q_weight=qw, k_weight=kw, rope_cos=cos,
                           rope_sin=sin, rope_form="even_cos_odd_sin")
    (gq, gk, gv), _ = ops.qkv_prologue(q.cuda(), k.cuda(), v.cuda(), num_heads=H, norm="rms_all_heads",
                                       q_weight=qw.cuda(), k_weight=kw.cuda(), rope_cos=cos.cuda(),
                                       rope_sin=sin.cuda(), rope_form="even_cos_odd_sin")
    _close_after_norm(gq, ref[0], dtype)
    _close_after_norm(gk, ref[1], dtype)
    assert torch.equal(gv.cpu(), ref[2])


def test_cogvideox_layer_norm_text_first(ops):
    dtype, H, D, St, Sv, bs = torch.bfloat16, 3, 64, 32, 200, 64
    S = St + Sv
    q, k, v = _proj(1, S, H * D, dtype, 14)
    g = torch.Generator().manual_seed(15)
    qw, qb, kw, kb = [(0.1 * torch.randn(D, generator=g) + (1 if i % 2 == 0 else 0)).to(dtype) for i in range(4)]
    cos, sin = _tables(Sv, D, 16)
    ref = orc.qkv_prologue(q, k, v, num_heads=H, norm="layer", q_weight=qw, q_bias=qb, k_weight=kw, k_bias=kb,
                           eps=1e-6, rope_cos=cos, rope_sin=sin, rope_range=(St, S))
    (gq, gk, gv), (pq, pk) = ops.qkv_prologue(q.cuda(), k.cuda(), v.cuda(), num_heads=H, norm="layer",
                                              q_weight=qw.cuda(), q_bias=qb.cuda(), k_weight=kw.cuda(),
                                              k_bias=kb.cuda(), eps=1e-6, rope_cos=cos.cuda(), rope_sin=sin.cuda(),
                                              rope_range=(St, S), pool_block_size=bs)
    _close_after_norm(gq, ref[0], dtype)
    _close_after_norm(gk, ref[1], dtype)
    assert torch.equal(gv.cpu(), ref[2])
    assert torch.equal(pq, ops.pool_blocks(gq, bs)) and torch.equal(pk, ops.pool_blocks(gk, bs))


def test_rejects_bad_arguments(ops):
    q, k, v = [t.cuda() for t in _proj(1, 64, 2 * 128, torch.bfloat16, 17)]
    cos, sin = [t.cuda() for t in _tables(64, 128, 18)]
    with pytest.raises(ValueError):          # block means from a row that is not a block boundary
        ops.qkv_prologue(q, k, v, num_heads=2, total_tokens=200, dst_row0=3, pool_block_size=64)
    with pytest.raises(ValueError):          # rows do not fit
        ops.qkv_prologue(q, k, v, num_heads=2, total_tokens=100, dst_row0=64)
    with pytest.raises(ValueError):
        ops.qkv_prologue(q, k, v, num_heads=2, rope_cos=cos)
    with pytest.raises(ValueError):          # head_dim 32
        ops.qkv_prologue(q, k, v, num_heads=8)
    with pytest.raises(ValueError):
        ops.qkv_prologue(q.cpu(), k.cpu(), v.cpu(), num_heads=2)


def test_prologue_feeds_the_state_machine(ops):
    """Projections -> prologue -> SparseAttentionWithMap with the prologue's block means handed over as
    `pooled_qk`: mask and output equal the ones of a call that pools the stored tensors itself."""
    import logging

    import MoD.mod.attn_mask as am
    from MoD.mod.state import create_adaptive_mask_state
    from moddit_b200 import synth

    H, grid, D, bs, text = 2, (4, 16, 16), 128, 128, 128
    q, k, v = synth.make_qkv(heads=H, grid=grid, head_dim=D, text_tokens=text, seed=5, device=torch.device("cuda"))
    video = grid[0] * grid[1] * grid[2]
    proj = [t[0].transpose(0, 1).reshape(1, video + text, H * D).contiguous() for t in (q, k, v)]   # token-major
    (pq, pk, pv), pools = ops.qkv_prologue(*proj, num_heads=H, pool_block_size=bs)
    assert torch.equal(pq, q) and torch.equal(pk, k) and torch.equal(pv, v)
    log = logging.getLogger("prologue-test")
    results = []
    for pooled in (None, pools):
        state = create_adaptive_mask_state("hunyuan", H, video, text, grid[1] * grid[2], grid[0], warmup_steps=2,
                                           top_k=6, predict_T=5, block_size=bs)
        state["score_producer"] = "pooled"
        for step in range(3):
            kw = {} if pooled is None else {"pooled_qk": pooled}
            out, _ = am.SparseAttentionWithMap(pq, pk, pv, state, log, current_step=step, **kw)
        results.append((state["mask"].clone(), out.clone()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
