"""Dense attention plus the exact video-video block sparsity map.

Public names and behaviour follow MoD/mod/triton_flash_sparsity.py:101-341; the module name is kept
for import compatibility although nothing here uses Triton.  Pass 1 is this build's own flash forward
(all key tiles kept, log-sum-exp returned); pass 2 replays QK^T on the tensor cores and counts
probabilities below the threshold.
"""
import math
import os
from typing import Tuple

import torch

from MoD.mod.cuda_flash_sparsity import cuda_backend_supported, cuda_sparsity_map
from moddit_b200 import ops as _ops


def _video_layout(model_type: str, sequence_length: int, video_token_num: int, text_token_num: int,
                  block_size: int) -> Tuple[int, int, int]:
    """(video_blocks, q_token_offset, k_token_offset) for the three token layouts."""
    if model_type == "wan":
        if video_token_num not in (0, sequence_length):
            raise ValueError(
                f"wan expects video_token_num to be 0 or S={sequence_length}, got {video_token_num}")
        return sequence_length // block_size, 0, 0
    if model_type == "hunyuan":
        return video_token_num // block_size, 0, 0
    if model_type == "cogvideox":
        return video_token_num // block_size, text_token_num, text_token_num
    raise ValueError(f"Unknown model_type: {model_type}, expected 'wan', 'hunyuan', or 'cogvideox'")


def _validate_inputs(query, key, value, threshold, block_size, model_type, video_token_num,
                     text_token_num) -> Tuple[float, int, int, int]:
    """Checks of MoD/mod/triton_flash_sparsity.py:123-178; returns (threshold, video_blocks, q_off, k_off)."""
    if query.ndim != 4:
        raise ValueError(f"query must have shape [B, H, S, D], got {tuple(query.shape)}")
    if key.shape != query.shape or value.shape != query.shape:
        raise ValueError("query, key, and value must have identical [B, H, S, D] shapes")
    if not (query.is_cuda and key.is_cuda and value.is_cuda):
        raise ValueError("query, key, and value must be CUDA tensors")
    if query.device != key.device or query.device != value.device:
        raise ValueError("query, key, and value must be on the same CUDA device")
    if query.dtype != key.dtype or query.dtype != value.dtype:
        raise ValueError("query, key, and value must have the same dtype")
    if query.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"expected float16 or bfloat16 inputs, got {query.dtype}")
    if block_size not in (64, 128):
        raise ValueError(f"block_size must be 64 or 128, got {block_size}")
    sequence_length, head_dim = query.shape[2], query.shape[3]
    if head_dim not in (64, 128):
        raise ValueError(f"head_dim must be 64 or 128, got {head_dim}")
    if model_type == "wan":
        video_tokens = sequence_length
    else:
        if video_token_num <= 0:
            raise ValueError(f"video_token_num must be positive for {model_type}")
        video_tokens = video_token_num
    if video_tokens % block_size:
        raise ValueError(f"video_token_num={video_tokens} must be divisible by block_size={block_size}")
    if text_token_num < 0:
        raise ValueError("text_token_num must be non-negative")
    if model_type in ("hunyuan", "cogvideox") and video_token_num + text_token_num > sequence_length:
        raise ValueError("video and text regions exceed the sequence length")
    if torch.is_tensor(threshold):
        if threshold.numel() != 1:
            raise ValueError("threshold tensor must contain one element")
        threshold_value = float(threshold.detach().item())
    else:
        threshold_value = float(threshold)
    if math.isnan(threshold_value):
        raise ValueError("threshold must not be NaN")
    video_blocks, q_offset, k_offset = _video_layout(model_type, sequence_length, video_token_num,
                                                     text_token_num, block_size)
    return threshold_value, video_blocks, q_offset, k_offset


def _triton_sparsity_map(query, key, lse, *, softmax_scale, log_threshold, q_video_offset, k_video_offset,
                         video_blocks, block_size) -> torch.Tensor:
    """Kept for callers of the reference's Triton entry point; runs the same sm_100a replay kernel."""
    return _ops.replay_map(query, key, lse, softmax_scale=float(softmax_scale), log_threshold=float(log_threshold),
                           q_video_offset=int(q_video_offset), k_video_offset=int(k_video_offset),
                           video_blocks=int(video_blocks), block_size=int(block_size))


def _compute_sparsity_map(query, key, lse, *, softmax_scale, log_threshold, q_video_offset, k_video_offset,
                          video_blocks, block_size) -> torch.Tensor:
    """Validates MOD_DIT_SPARSITY_BACKEND as the reference does (auto | cuda | triton); every accepted
    value runs the one sm_100a kernel, and an unsupported device is an error rather than a fallback."""
    backend = os.environ.get("MOD_DIT_SPARSITY_BACKEND", "auto").lower()
    if backend not in {"auto", "cuda", "triton"}:
        raise ValueError("MOD_DIT_SPARSITY_BACKEND must be one of: auto, cuda, triton")
    if not cuda_backend_supported(query.device if query.is_cuda else None):
        raise RuntimeError("the sparsity-map replay needs an sm_100 GPU (no other backend exists)")
    kwargs = dict(softmax_scale=softmax_scale, log_threshold=log_threshold, q_video_offset=q_video_offset,
                  k_video_offset=k_video_offset, video_blocks=video_blocks, block_size=block_size)
    if backend == "triton":
        return _triton_sparsity_map(query, key, lse, **kwargs)
    return cuda_sparsity_map(query, key, lse, **kwargs)


_DENSE_LISTS = {}


def _dense_lists(device: torch.device, sequence_length: int):
    """All-kept work lists for a sequence length (cached per device)."""
    key = (device.index, sequence_length)
    hit = _DENSE_LISTS.get(key)
    if hit is None:
        nb = (sequence_length + 127) // 128
        mask = torch.ones(1, nb, nb, device=device, dtype=torch.bool)
        hit = _ops.tile_lists(mask, 128, sequence_length)
        _DENSE_LISTS[key] = hit
    return hit


def dense_attention_with_lse(query, key, value, softmax_scale=None, kv_len=None):
    """Dense flash forward of (B,H,S,D) tensors; returns (O, LSE (B,H,S) float32 natural log)."""
    counts, entries = _dense_lists(query.device, query.shape[2])
    return _ops.sparse_attn_fwd(query, key, value, counts, entries, softmax_scale=softmax_scale,
                                kv_len_lo=kv_len, kv_len_hi=kv_len, return_lse=True, check_status=False)


@torch.no_grad()
def flash_attn_with_sparsity_map(query, key, value, threshold, block_size, model_type="hunyuan",
                                 video_token_num=0, text_token_num=0) -> Tuple[torch.Tensor, torch.Tensor]:
    """(B,H,S,D) fp16/bf16 -> (O (B,H,S,D), sparsity map (B,H,video_blocks,video_blocks) fp16).

    Same contract as MoD/mod/triton_flash_sparsity.py:275-341.
    """
    threshold_value, video_block_num, q_video_offset, k_video_offset = _validate_inputs(
        query, key, value, threshold, block_size, model_type, video_token_num, text_token_num)
    D = query.shape[3]
    query, key, value = query.contiguous(), key.contiguous(), value.contiguous()
    sm_scale = D ** -0.5
    out, lse = dense_attention_with_lse(query, key, value, sm_scale)
    ln_thresh = math.log(threshold_value) if threshold_value > 0 else float("-inf")
    sparsity_map = _compute_sparsity_map(
        query, key, lse, softmax_scale=sm_scale, log_threshold=ln_thresh, q_video_offset=q_video_offset,
        k_video_offset=k_video_offset, video_blocks=video_block_num, block_size=block_size)
    return out, sparsity_map
