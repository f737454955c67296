"""Block grid of the sequence: the product's `block_geometry` equals the oracle's, reduces to the reference's floor
divisions on block-aligned shapes, and gives the stated grid for the CogVideoX-1.5 shape of the specification."""
from oracle import moddit_oracle as orc


def test_block_geometry_matches_oracle_and_reference_on_aligned_shapes():
    from MoD.mod.attn_mask import block_geometry
    cases = [("cogvideox", 64, 44880, 224, 45104), ("cogvideox", 64, 1024, 128, 1152), ("hunyuan", 128, 115200, 256, 115456),
             ("hunyuan", 64, 1000, 100, 1100), ("wan", 128, 69120, 0, 69120), ("wan", 64, 1000, 0, 1000),
             ("cogvideox", 128, 816, 40, 856)]
    for c in cases:
        assert block_geometry(*c) == orc.block_geometry(*c), c
    assert block_geometry("cogvideox", 64, 44880, 224, 45104) == (705, 701, 4)
    # aligned shapes: the reference's floor divisions
    assert block_geometry("cogvideox", 64, 1024, 128, 1152) == (1152 // 64, 1024 // 64, 128 // 64)
    assert block_geometry("hunyuan", 128, 115200, 256, 115456) == (902, 900, 0)


def test_pair_order_is_a_longest_first_permutation_per_group():
    """The oracle's start order of the sparse forward's work items: every group's part is a permutation of the
    group's own items, its first entries are the two longest pairs of each head, the rest runs head after head
    with non-increasing list lengths (ties by index)."""
    import numpy as np
    from oracle import moddit_oracle as orc
    rng = np.random.default_rng(3)
    for Hm, npairs, hpg in ((1, 1, None), (5, 7, None), (5, 7, 2), (6, 9, 3), (4, 3, 1), (3, 2, 2)):
        counts = rng.integers(0, 6, size=(Hm, npairs))
        order = orc.pair_order(counts, hpg)
        g_size = Hm if hpg is None else hpg
        for g0 in range(0, Hm, g_size):
            Hg = min(g_size, Hm - g0)
            part = order[g0 * npairs:(g0 + Hg) * npairs]
            assert sorted(part.tolist()) == list(range(Hg * npairs))
            r0 = min(2, npairs)
            for hl in range(Hg):
                lens = counts[g0 + hl]
                mine = [int(part[r * Hg + hl]) for r in range(r0)]
                mine += part[r0 * Hg + hl * (npairs - r0): r0 * Hg + (hl + 1) * (npairs - r0)].tolist()
                assert all(i // npairs == hl for i in mine)
                keys = [(-int(lens[i % npairs]), i % npairs) for i in mine]
                assert keys == sorted(keys)

