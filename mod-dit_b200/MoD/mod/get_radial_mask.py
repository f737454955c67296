"""Static radial block mask for `--sparse_type radial` (the reference's MoD/mod/get_radial_mask.py).

Only the entry point the attention path calls is provided: `get_radial_mask`, same arguments and result
as the reference (:157-164).  The reference builds token-level band masks for every pair of frames and
shrinks them to blocks on the host side of torch; here one CUDA kernel decides every block in closed form
(`moddit_radial_mask`), with identical results.
"""
import torch

from moddit_b200 import ops as _ops


def get_radial_mask(query: torch.Tensor, video_token_num: int, num_frame: int, block_size: int = 128,
                    decay_factor: float = 0.2, model_type: str = None) -> torch.Tensor:
    """(num_heads, S//block_size, S//block_size) bool mask for a (B, H, S, D) query; every head shares one
    mask (an expanded view, not H copies).  Raises ValueError for model types other than hunyuan and wan."""
    num_head, seq_len = query.size(1), query.size(2)
    mask = _ops.radial_mask(model_type, video_token_num, num_frame, seq_len, query.device, block_size=block_size,
                            decay_factor=decay_factor)
    return mask.unsqueeze(0).expand(num_head, -1, -1)
