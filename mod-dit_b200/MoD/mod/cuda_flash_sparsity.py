"""Exact sparsity-map replay on the sm_100a tcgen05 kernel.

Keeps the names of the reference loader (MoD/mod/cuda_flash_sparsity.py:56-104).  The kernel lives in
the ahead-of-time built C-ABI library, so there is nothing to JIT: importing this module fails loudly
if the library is missing.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from moddit_b200 import ops as _ops


def cuda_backend_supported(device: Optional[Union[torch.device, int]] = None) -> bool:
    """Whether `device` can run the replay kernel (compute capability 10.x)."""
    if not torch.cuda.is_available():
        return False
    if device is None:
        device = torch.cuda.current_device()
    device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
    if device.type != "cuda":
        return False
    major, _ = torch.cuda.get_device_capability(device)
    return major == 10


def cuda_sparsity_map(
    query: torch.Tensor,
    key: torch.Tensor,
    lse: torch.Tensor,
    *,
    softmax_scale: float,
    log_threshold: float,
    q_video_offset: int,
    k_video_offset: int,
    video_blocks: int,
    block_size: int,
) -> torch.Tensor:
    """FP16 (B, H, video_blocks, video_blocks) map: count(S < lse + log_threshold) / block_size^2.

    Same contract as the reference's pybind `sparsity_map` (MoD/mod/cuda_flash_sparsity_kernel.cu:258-334):
    contiguous (B,H,S,D) fp16/bf16 Q and K, contiguous float32 (B,H,S) LSE, RuntimeError on bad input,
    launch on the current stream of the inputs' device.
    """
    if not cuda_backend_supported(query.device if query.is_cuda else None):
        capability = torch.cuda.get_device_capability(query.device) if query.is_cuda else None
        raise RuntimeError(f"CUDA sparsity backend requires an sm_100 GPU, got {capability}")
    return _ops.replay_map(
        query, key, lse,
        softmax_scale=float(softmax_scale),
        log_threshold=float(log_threshold),
        q_video_offset=int(q_video_offset),
        k_video_offset=int(k_video_offset),
        video_blocks=int(video_blocks),
        block_size=int(block_size),
    )


def extension_error() -> Optional[BaseException]:
    """The reference exposes a cached JIT build error here; an ahead-of-time library has none."""
    return None
