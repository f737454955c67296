"""Seeded synthetic q/k/v with spatio-temporal locality, standing in for video-DiT activations.

Video token p sits at (t, y, x) of a T x Hh x Ww latent grid, row-major.  pe(p) is a 48-dim vector:
3 axes x 8 octave frequencies x {sin, cos} of the normalised coordinate.  Per head,
    q = 0.5 * N(0,1) + gain * pe @ W_q,   k = 0.5 * N(0,1) + gain * pe @ W_k,   v = N(0,1)
with W_q ~ N(0, 1/48) and W_k = corr * W_q + sqrt(1 - corr^2) * N(0, 1/48).  `corr` > 0 is what makes
nearby tokens attend to each other (independent W_q and W_k give no locality).  Text tokens are N(0,1).
`axis_mix` (per head weights of the t / y / x parts of pe) gives head-varying patterns: weight on x
only produces vertical stripes, on t only temporal diagonals.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch


def positional_code(T: int, Hh: int, Ww: int, device, dtype=torch.float32) -> torch.Tensor:
    """(T*Hh*Ww, 48) sinusoid code; columns [0,16) t, [16,32) y, [32,48) x."""
    t, y, x = torch.meshgrid(torch.arange(T, device=device), torch.arange(Hh, device=device),
                             torch.arange(Ww, device=device), indexing="ij")
    pos = torch.stack([t.flatten() / max(T, 1), y.flatten() / Hh, x.flatten() / Ww], 1).to(dtype)
    freqs = (2.0 ** torch.arange(8, device=device)).to(dtype)
    ang = pos[:, :, None] * freqs[None, None, :] * math.pi
    return torch.cat([ang.sin(), ang.cos()], -1).reshape(pos.shape[0], 48)


def make_qkv(*, heads: int, grid: Tuple[int, int, int], head_dim: int, text_tokens: int = 0,
             text_first: bool = False, seed: int = 0, gain: float = 2.0, corr: float = 1.0,
             axis_mix: Optional[Sequence[Sequence[float]]] = None, device="cuda", dtype=torch.bfloat16,
             head_begin: int = 0, head_end: Optional[int] = None):
    """Returns q, k, v of shape (1, head_end-head_begin, T*Hh*Ww + text_tokens, head_dim) on `device`.

    Head h is generated from its own generator seeded with seed * 4096 + h, so any subset of heads
    (a rank's shard) reproduces the same values as the full tensor.
    """
    device = torch.device(device)
    T, Hh, Ww = grid
    nv = T * Hh * Ww
    N = nv + text_tokens
    head_end = heads if head_end is None else head_end
    hl = head_end - head_begin
    pe = positional_code(T, Hh, Ww, device)
    q = torch.empty(1, hl, N, head_dim, device=device, dtype=dtype)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    v0 = text_tokens if text_first else 0
    t0 = 0 if text_first else nv
    for h in range(head_begin, head_end):
        g = torch.Generator(device=device).manual_seed(seed * 4096 + h)
        i = h - head_begin
        wq = torch.randn(48, head_dim, generator=g, device=device) / math.sqrt(48.0)
        wn = torch.randn(48, head_dim, generator=g, device=device) / math.sqrt(48.0)
        wk = corr * wq + math.sqrt(max(0.0, 1.0 - corr * corr)) * wn
        if axis_mix is not None:
            mix = torch.tensor(axis_mix[h % len(axis_mix)], device=device, dtype=torch.float32)
            scale = mix.repeat_interleave(16).unsqueeze(-1)                            # (48, 1)
            wq, wk = wq * scale, wk * scale
        for dst, w in ((q, wq), (k, wk)):
            x = 0.5 * torch.randn(nv, head_dim, generator=g, device=device) + gain * (pe @ w)
            dst[0, i, v0:v0 + nv] = x.to(dtype)
        v[0, i, v0:v0 + nv] = torch.randn(nv, head_dim, generator=g, device=device).to(dtype)
        if text_tokens:
            for dst in (q, k, v):
                dst[0, i, t0:t0 + text_tokens] = torch.randn(text_tokens, head_dim, generator=g,
                                                             device=device).to(dtype)
    return q, k, v


WORKLOADS = {
    # name: model_type, heads, head_dim, block, grid (T,Hh,Ww), text tokens, text first, top_k, predict_T
    "hunyuan": dict(model_type="hunyuan", heads=24, head_dim=128, block_size=128, grid=(30, 48, 80),
                    text_tokens=256, text_first=False, top_k=300, predict_T=5),
    "wan": dict(model_type="wan", heads=40, head_dim=128, block_size=128, grid=(18, 48, 80), text_tokens=0,
                text_first=False, top_k=200, predict_T=10),
    "cogvideox": dict(model_type="cogvideox", heads=48, head_dim=64, block_size=64, grid=(11, 48, 84),
                      text_tokens=256, text_first=True, top_k=100, predict_T=5),
    "medium": dict(model_type="hunyuan", heads=8, head_dim=128, block_size=128, grid=(8, 64, 64), text_tokens=256,
                   text_first=False, top_k=80, predict_T=5),
    "small": dict(model_type="hunyuan", heads=4, head_dim=128, block_size=128, grid=(8, 32, 32), text_tokens=256,
                  text_first=False, top_k=30, predict_T=5),
}
