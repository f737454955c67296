"""ctypes binding of libmoddit.so (the C ABI declared in include/moddit.h).

The library is built in-tree by `csrc/build.py`.  There is no fallback: if the shared object is
missing or a symbol cannot be resolved, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
# MODDIT_LIB_PATH lets a developer load another build of the same ABI (e.g. an instrumented one)
LIB_PATH = os.environ.get("MODDIT_LIB_PATH") or os.path.join(_HERE, "libmoddit.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: build it with `python mod-dit_b200/csrc/build.py` (needs nvcc; there is no "
        "fallback implementation)")

lib = ctypes.CDLL(LIB_PATH)

# name -> (restype, argtypes); mirrors include/moddit.h declaration by declaration
SIGNATURES = {
    "moddit_abi_version": (c_int, []),
    "moddit_last_error_string": (c_char_p, []),
    "moddit_pool_blocks": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moddit_pool_blocks_shard": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "moddit_qkv_prologue_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "moddit_qkv_prologue": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_int,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                                    c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                    c_int, c_void_p, c_size_t, c_void_p]),
    "moddit_pooled_map": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_void_p, c_void_p]),
    "moddit_pooled_map_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "moddit_pooled_map_ws": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                     c_void_p, c_void_p, c_size_t, c_void_p]),
    "moddit_replay_map": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_float, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moddit_replay_map_mma": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                      c_float, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moddit_replay_status": (c_int, [c_void_p, c_void_p]),
    "moddit_mts_workspace_bytes": (c_size_t, [c_int, c_int]),
    "moddit_mts": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_int, c_int, c_int,
                           c_void_p, c_void_p, c_size_t, c_void_p]),
    "moddit_mts_noalloc_max_bytes": (c_size_t, []),
    "moddit_mts_noalloc": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moddit_mtm": (c_int, [c_int, c_int, c_float, c_void_p, c_void_p]),
    "moddit_reconstruct_map": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moddit_solve_factor_bytes": (c_size_t, [c_int]),
    "moddit_solve_prepare_workspace_bytes": (c_size_t, [c_int]),
    "moddit_solve_prepare": (c_int, [c_int, c_int, c_double, c_void_p, c_void_p, c_size_t, c_void_p]),
    "moddit_solve_workspace_bytes": (c_size_t, [c_int, c_int]),
    "moddit_solve": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_double, c_void_p, c_void_p, c_size_t,
                             c_void_p]),
    "moddit_solve_small_max_n": (c_int, []),
    "moddit_solve_small_factor_bytes": (c_size_t, [c_int]),
    "moddit_solve_small_prepare": (c_int, [c_int, c_int, c_float, c_void_p, c_void_p]),
    "moddit_solve_small": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "moddit_select_lines": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                    c_void_p, c_void_p]),
    "moddit_head_modes": (c_int, [c_void_p, c_int, c_float, c_void_p, c_void_p]),
    "moddit_radial_mask": (c_int, [c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "moddit_mask_from_lines": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p, c_void_p]),
    "moddit_select_mass": (c_int, [c_void_p, c_int, c_int, c_float, c_void_p, c_void_p]),
    "moddit_block_similarity": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "moddit_select_topk_blocks": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "moddit_tile_lists": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_void_p, c_void_p]),
    "moddit_order_pairs": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moddit_copy_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "moddit_copy_rows_dma": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "moddit_copy_rows_multi": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "moddit_copy_rows_narrow": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
    "moddit_sparse_attn_fwd_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                               c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_void_p,
                                               c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "moddit_sparse_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
                                       c_void_p, c_void_p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here means the library is stale: rebuild it
    _fn.restype = _res
    _fn.argtypes = _args

MODDIT_BF16, MODDIT_FP16 = 0, 1
NORM_KIND = {None: 0, "none": 0, "rms_head": 1, "rms_all_heads": 2, "layer": 3}
ROPE_FORM = {"elementwise": 0, "even_cos_odd_sin": 1, "pair": 2}
LAYOUT = {"wan": 0, "hunyuan": 1, "cogvideox": 2}
MODE_SPARSE, MODE_BLOCK_DIAGONAL, MODE_FULL = 0, 1, 2
MODE_CODE = {"sparse": MODE_SPARSE, "block_diagonal": MODE_BLOCK_DIAGONAL, "full": MODE_FULL}
MODE_NAME = {v: k for k, v in MODE_CODE.items()}


class ModditError(RuntimeError):
    """A C-ABI call returned a negative status."""


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib.moddit_last_error_string().decode("utf-8", "replace")
        if rc == -1:
            raise ValueError(f"{what}: {msg}")
        raise ModditError(f"{what} failed with code {rc}: {msg}")
