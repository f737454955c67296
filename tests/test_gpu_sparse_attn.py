"""GPU parity of the block-sparse flash-attention forward against fp32 block-masked attention.

Tolerance (stated by the build specification for 16-bit inputs against fp32 masked attention):
max-abs <= 2e-2 and relative L2 <= 1e-2.
"""
import pytest
import torch

from oracle import moddit_oracle as orc

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
REL_L2 = 1e-2


@pytest.fixture(scope="module")
def ops():
    from moddit_b200 import ops as _ops
    return _ops


def _check(out, ref):
    out = out.float().cpu()
    assert torch.isfinite(out).all()
    err = (out - ref).abs().max().item()
    rel = ((out - ref).norm() / ref.norm().clamp_min(1e-12)).item()
    assert err <= MAX_ABS, f"max-abs {err}"
    assert rel <= REL_L2, f"rel-l2 {rel}"


def _run(ops, *, D, dtype, bs, N, H, density, seed, B=1, Hm=None, q_split=None, kv_lo=None, kv_hi=None,
         qk_gain=1.0, ensure_diag=True):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, N, D, generator=g) * qk_gain).to(dtype)
    k = (torch.randn(B, H, N, D, generator=g) * qk_gain).to(dtype)
    v = torch.randn(B, H, N, D, generator=g).to(dtype)
    nb = (N + bs - 1) // bs
    Hm = H if Hm is None else Hm
    mask = torch.rand(Hm, nb, nb, generator=g) < density
    if ensure_diag:
        idx = torch.arange(nb)
        mask[:, idx, idx] = True
    lists = ops.tile_lists(mask.cuda(), bs, N)
    counts, entries = lists
    # alternate between index order and the longest-first order: results must not depend on it
    out, lse = ops.sparse_attn_fwd(q.cuda(), k.cuda(), v.cuda(), counts, entries, order=lists.order if seed % 2 else None,
                                   q_split=q_split, kv_len_lo=kv_lo, kv_len_hi=kv_hi, return_lse=True)
    refs, lses = [], []
    for b in range(B):
        r, l = orc.masked_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], mask if Hm == H else mask.repeat(H // Hm, 1, 1),
                                    bs, q_split=q_split, kv_len_lo=kv_lo, kv_len_hi=kv_hi, return_lse=True)
        refs.append(r)
        lses.append(l)
    ref, ref_lse = torch.cat(refs), torch.cat(lses)
    _check(out, ref)
    lse = lse.cpu()
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin)
    assert (lse[fin] - ref_lse[fin]).abs().max().item() <= 5e-3
    return out


def test_smallest_dense_tile(ops):
    """One CTA, one key tile, both query tiles: the minimal exercise of QK^T, softmax, PV."""
    _run(ops, D=128, dtype=torch.bfloat16, bs=128, N=256, H=1, density=1.1, seed=0)


def test_single_query_tile(ops):
    _run(ops, D=128, dtype=torch.bfloat16, bs=128, N=128, H=1, density=1.1, seed=1)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dense_multi_tile(ops, D, dtype):
    _run(ops, D=D, dtype=dtype, bs=128, N=1024, H=2, density=1.1, seed=2)


@pytest.mark.parametrize("D,bs", [(128, 128), (64, 64), (128, 64), (64, 128)])
def test_sparse_masks(ops, D, bs):
    _run(ops, D=D, dtype=torch.bfloat16, bs=bs, N=1536, H=3, density=0.3, seed=3)


def test_odd_tile_count_and_ragged_tail(ops):
    _run(ops, D=128, dtype=torch.bfloat16, bs=128, N=128 * 5, H=2, density=0.5, seed=4)
    _run(ops, D=128, dtype=torch.bfloat16, bs=128, N=1000, H=2, density=0.5, seed=5)
    _run(ops, D=64, dtype=torch.bfloat16, bs=64, N=64 * 9 + 17, H=2, density=0.5, seed=6)


def test_rows_without_kept_blocks_give_zeros(ops):
    out = _run(ops, D=128, dtype=torch.bfloat16, bs=128, N=768, H=2, density=0.25, seed=7, ensure_diag=False)
    assert torch.isfinite(out.float()).all()


def test_text_layout_key_limits(ops):
    """Hunyuan-style: video rows see keys below a 64-rounded border, text rows only the valid keys."""
    N, video = 128 * 6 + 256, 128 * 6
    valid = video + 77
    border = min(N, (valid + 63) // 64 * 64)
    _run(ops, D=128, dtype=torch.bfloat16, bs=128, N=N, H=2, density=0.4, seed=8, q_split=video, kv_lo=border,
         kv_hi=valid)


def test_mask_heads_broadcast_over_batch(ops):
    _run(ops, D=64, dtype=torch.float16, bs=64, N=512, H=2, B=2, Hm=2, density=0.5, seed=9)


def test_large_logits_exercise_rescaling(ops):
    """Row maxima that grow a lot from tile to tile force the accumulator rescale path."""
    _run(ops, D=128, dtype=torch.bfloat16, bs=128, N=2048, H=1, density=1.1, seed=10, qk_gain=3.0)


def test_two_calls_are_bitwise_identical(ops):
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(1, 2, 1024, 128, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    mask = (torch.rand(2, 8, 8, generator=g) < 0.5).cuda()
    lists = ops.tile_lists(mask, 128, 1024)
    counts, entries = lists
    a = ops.sparse_attn_fwd(q, k, v, counts, entries)
    b = ops.sparse_attn_fwd(q, k, v, counts, entries)
    c = ops.sparse_attn_fwd(q, k, v, counts, entries, order=lists.order)
    assert torch.equal(a, b) and torch.equal(a, c)
    # the start order is a permutation of all (head, pair) items: the two longest pairs of every head first,
    # then head after head with non-increasing list lengths
    cnt = counts.cpu()
    Hm, npairs = cnt.shape
    o = lists.order.cpu().long().flatten()
    assert sorted(o.tolist()) == list(range(Hm * npairs))
    flat = cnt.flatten()
    for h in range(Hm):
        top2 = sorted(cnt[h].tolist(), reverse=True)[:2]
        assert [int(flat[o[r * Hm + h]]) for r in range(2)] == top2 and all(int(o[r * Hm + h]) // npairs == h for r in range(2))
        rest = o[2 * Hm + h * (npairs - 2): 2 * Hm + (h + 1) * (npairs - 2)]
        assert (rest // npairs == h).all()
        assert (flat[rest][:-1] >= flat[rest][1:]).all()


def test_medium_shape_against_chunked_oracle(ops):
    """8k tokens, 4 heads, reference-like mask structure (columns + diagonals + per-frame blocks)."""
    N, H, bs, D = 8192, 4, 128, 128
    n = N // bs
    g = torch.Generator().manual_seed(12)
    lines = torch.stack([torch.randperm(3 * n - 1, generator=g)[:20] for _ in range(H)])
    mask = orc.generate_mask_from_lines(model_type="wan", block_size=bs, video_token_num=N, text_token_num=0,
                                        seq_len=N, blocks_per_frame=8, selected_lines=lines,
                                        mode=["block_diagonal"] * H)
    q, k, v = (torch.randn(1, H, N, D, generator=g).to(torch.bfloat16) for _ in range(3))
    counts, entries = ops.tile_lists(mask.cuda(), bs, N)
    out = ops.sparse_attn_fwd(q.cuda(), k.cuda(), v.cuda(), counts, entries)
    ref = orc.masked_attention(q, k, v, mask, bs)
    _check(out, ref)


def test_head_groups_give_the_same_output_as_one_launch(ops):
    """One launch per group of heads over slices of the lists (order made group by group) against one launch."""
    from MoD.mod.attn_mask import AttentionSparseEngine
    torch.manual_seed(7)
    H, N, D, bs = 5, 1536, 128, 128
    q, k, v = (torch.randn(1, H, N, D, device="cuda").bfloat16() for _ in range(3))
    mask = torch.rand(H, N // bs, N // bs, device="cuda") < 0.35
    idx = torch.arange(N // bs, device="cuda")
    mask[:, idx, idx] = True
    whole = ops.tile_lists(mask, bs, N)
    assert torch.equal(whole.order.view(-1).cpu(), torch.from_numpy(orc.pair_order(whole.counts.cpu().numpy())))
    ref = AttentionSparseEngine(q, k, v, mask, block_size=bs, _lists=whole)
    for groups in (2, 3, 5):
        hpg = (H + groups - 1) // groups
        lists = ops.tile_lists(mask, bs, N, heads_per_group=hpg)
        npairs = lists.counts.shape[1]
        live = torch.arange(lists.entries.shape[-1], device="cuda")[None, None, :] < whole.counts[:, :, None]
        assert torch.equal(lists.counts, whole.counts) and torch.equal(lists.entries[live], whole.entries[live])
        flat = lists.order.view(-1)
        for g in range(groups):                               # every group's order is a permutation of its own items
            h0, h1 = g * hpg, min(H, (g + 1) * hpg)
            if h0 < h1:
                part = flat[h0 * npairs:h1 * npairs].sort().values
                assert torch.equal(part, torch.arange((h1 - h0) * npairs, device="cuda", dtype=torch.int32))
        assert torch.equal(flat.cpu(), torch.from_numpy(orc.pair_order(whole.counts.cpu().numpy(), hpg)))
        ev = torch.cuda.Event()
        ev.record()
        ready = [ev if g % 2 == 0 else None for g in range(groups)]
        out = AttentionSparseEngine(q, k, v, mask, block_size=bs, _lists=lists, _group_ready=ready)
        torch.cuda.synchronize()
        assert torch.equal(out, ref), groups
    ops.raise_on_status(q.device)

