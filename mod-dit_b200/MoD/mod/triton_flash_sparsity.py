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
    """The reference's second replay kernel (Triton, :28-98,181-225).  Nothing here uses Triton: the name runs
    this library's second, independently written replay kernel (warp-level mma.sync products from registers, no
    TMA and no tensor memory), so a caller that checks one replay path against the other - the reference's own test
    does - still compares two implementations."""
    return _ops.replay_map(query, key, lse, softmax_scale=float(softmax_scale), log_threshold=float(log_threshold),
                           q_video_offset=int(q_video_offset), k_video_offset=int(k_video_offset),
                           video_blocks=int(video_blocks), block_size=int(block_size), kernel="mma")


def _compute_sparsity_map(query, key, lse, *, softmax_scale, log_threshold, q_video_offset, k_video_offset,
                          video_blocks, block_size) -> torch.Tensor:
    """Validates MOD_DIT_SPARSITY_BACKEND as the reference does (auto | cuda | triton).  `auto` and `cuda` run the
    tcgen05 replay kernel, `triton` the second, independently written one (there is no Triton here); an unsupported
    device is an error rather than a fallback."""
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
                                kv_len_lo=kv_len, kv_len_hi=kv_len, return_lse=True, check_status="deferred")


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


# ---- self-test of the module (`python -m MoD.mod.triton_flash_sparsity`), as in the reference (:343-455) ----

@torch.no_grad()
def _naive_attn_with_sparsity(query, key, value, threshold, block_size, model_type="hunyuan", video_token_num=0,
                              text_token_num=0):
    """Checker for the self-test below, never used by the attention path: the full probability matrix with
    tensor expressions in float32 on the inputs' device, the output from it, and per video block the share of
    probabilities below the threshold (:345-370).  Memory grows with S^2: small sequences only."""
    B, H, S, D = query.shape
    if model_type not in ("hunyuan", "wan", "cogvideox"):
        raise ValueError(f"Unknown model_type: {model_type}")
    video = S if model_type == "wan" else video_token_num
    first = text_token_num if model_type == "cogvideox" else 0
    n = video // block_size
    probs = torch.softmax(query.float() @ key.float().transpose(-1, -2) * D ** -0.5, dim=-1)
    output = (probs @ value.float()).to(query.dtype)
    tiles = probs[:, :, first:first + video, first:first + video].reshape(B, H, n, block_size, n, block_size)
    return output, tiles.lt(threshold).float().mean(dim=(3, 5)).to(torch.float16)


def test_correctness(B=1, H=4, S=640, D=128, block_size=64, threshold=0.01, model_type="hunyuan"):
    """Output and map of the device path against the checker on seeded inputs; the reference's bounds (5e-2)."""
    g = torch.Generator(device="cuda").manual_seed(42)
    q, k, v = (torch.randn(B, H, S, D, device="cuda", dtype=torch.float16, generator=g) for _ in range(3))
    text = 128
    kw = dict(model_type=model_type, video_token_num=S - text, text_token_num=text)
    out, sp = flash_attn_with_sparsity_map(q, k, v, threshold, block_size, **kw)
    ref_out, ref_sp = _naive_attn_with_sparsity(q, k, v, threshold, block_size, **kw)
    o_err = (out.float() - ref_out.float()).abs().max().item()
    sp_err = (sp.float() - ref_sp.float()).abs().max().item()
    print(f"  O max error:        {o_err:.6f}")
    print(f"  Sparsity max error: {sp_err:.6f}")
    assert o_err < 5e-2, f"O error too large: {o_err}"
    assert sp_err < 5e-2, f"Sparsity error too large: {sp_err}"


def benchmark(B=1, H=24, S=4096, D=128, block_size=128, threshold=0.01, warmup=10, rep=50):
    """Milliseconds per call of the device path and of the checker (CUDA events on the current stream)."""
    q, k, v = (torch.randn(B, H, S, D, device="cuda", dtype=torch.float16) for _ in range(3))
    kw = dict(video_token_num=S - 128, text_token_num=128)

    def time_ms(fn):
        for _ in range(warmup):
            fn(q, k, v, threshold, block_size, **kw)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(rep):
            fn(q, k, v, threshold, block_size, **kw)
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / rep

    ours, naive = time_ms(flash_attn_with_sparsity_map), time_ms(_naive_attn_with_sparsity)
    print(f"  dense forward + replay map:    {ours:.2f} ms")
    print(f"  tensor expressions:            {naive:.2f} ms")
    print(f"  Speedup:                       {naive / ours:.1f}x")


if __name__ == "__main__":
    print("=== Correctness Tests ===")
    for _model in ("hunyuan", "cogvideox"):
        for _bs in (64, 128):
            print(f"model_type={_model}, block_size={_bs}, D=128")
            test_correctness(block_size=_bs, D=128, model_type=_model)
    print("\nAll correctness tests passed!\n")
    print("=== Benchmark (B=1, H=24, S=4096, D=128, block_size=128) ===")
    benchmark()
