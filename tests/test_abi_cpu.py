"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, rejects bad input."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "moddit.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moddit_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from moddit_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} declared in include/moddit.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert _lib.lib.moddit_abi_version() == 2


def test_argument_errors_do_not_touch_the_device():
    from moddit_b200 import _lib
    lib = _lib.lib
    assert lib.moddit_pool_blocks(None, 0, 1, 1, 64, 64, None, None) == -1
    assert b"null" in lib.moddit_last_error_string()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.moddit_pool_blocks(p, 0, 1, 128, 96, 64, p, None) == -2          # head_dim 96
    assert b"head_dim" in lib.moddit_last_error_string()
    assert lib.moddit_pool_blocks(p, 0, 1, 128, 64, 32, p, None) == -2          # block_size 32
    assert lib.moddit_mts(p, None, None, 0, 0, 0, None, 1, 8, 2, p, None, 0, None) == -4   # no workspace
    assert lib.moddit_solve_prepare(8, 2, 0.0, p, p, 1 << 20, None) == -1       # lambda must be positive
    assert lib.moddit_mts_workspace_bytes(24, 900) > 0
    assert lib.moddit_solve_factor_bytes(900) == 8 * (901 * 901 + 2 * 1799)
    assert lib.moddit_replay_map(p, p, p, 0, 1, 128, 64, 64, 0.125, -6.9, 0, 0, 3, p, None) == -1   # region too long
    assert b"exceeds sequence length" in lib.moddit_last_error_string()


def test_ops_reject_cpu_tensors():
    from moddit_b200 import ops
    x = torch.zeros(1, 1, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        ops.pool_blocks(x, 64)
    with pytest.raises(ValueError, match="CUDA"):
        ops.sparse_attn_fwd(x, x, x, torch.zeros(1, 1, dtype=torch.int32), torch.zeros(1, 1, 1, dtype=torch.int32))


def test_work_lists_survive_pickling_with_the_state_dict():
    """A state dict holds its mask and the work lists built from it; saving and loading it keeps the pairing
    (the cached lists are recognised by the identity of the mask tensor)."""
    import io

    from moddit_b200.ops import TileLists
    mask = torch.ones(2, 3, 3, dtype=torch.bool)
    lists = TileLists(torch.zeros(2, 1, dtype=torch.int32), torch.ones(2, 1, 3, dtype=torch.int32),
                      torch.arange(2, dtype=torch.int32).view(2, 1))
    state = {"mask": mask, "_tile_lists": (mask, lists), "mode": ["sparse", "full"], "features_history": []}
    buf = io.BytesIO()
    torch.save(state, buf)
    buf.seek(0)
    back = torch.load(buf, weights_only=False)
    assert isinstance(back["_tile_lists"][1], TileLists) and back["_tile_lists"][0] is back["mask"]
    counts, entries = back["_tile_lists"][1]
    assert torch.equal(counts, lists.counts) and torch.equal(entries, lists.entries)
    assert torch.equal(back["_tile_lists"][1].order, lists.order)
