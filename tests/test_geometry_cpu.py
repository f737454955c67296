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
