"""Seeded synthetic q/k/v with spatio-temporal locality, standing in for video-DiT activations.

Video token p sits at (t, y, x) of a T x Hh x Ww latent grid, row-major.  pe(p) is a 48-dim vector:
3 axes x 8 octave frequencies x {sin, cos} of the normalised coordinate.  Per head,
    q = 0.5 * N(0,1) + gain * pe @ W_q,   k = 0.5 * N(0,1) + gain * pe @ W_k,   v = N(0,1)
with W_q ~ N(0, 1/48) and W_k = corr * W_q + sqrt(1 - corr^2) * N(0, 1/48).  `corr` > 0 is what makes
nearby tokens attend to each other (independent W_q and W_k give no locality).  Text tokens are N(0,1).
`axis_mix` (per head weights of the t / y / x parts of pe, plus an optional fourth weight) gives head-varying
patterns.  All three axes: a local window around the diagonal.  y and x without t: the same place in every
frame, i.e. diagonals at multiples of one frame's blocks (temporal diagonals).  The fourth weight s adds a fixed
unit direction u to every query (s * u) and to the keys of one token block in `SINK_PERIOD` (s * u, blocks chosen
per head from its seed): keys every query attends to, i.e. vertical stripes.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

SINK_PERIOD = 16        # one block of SINK_BLOCK tokens in this many carries the stripe direction
SINK_BLOCK = 128


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
        sink = 0.0
        if axis_mix is not None:
            weights = list(axis_mix[h % len(axis_mix)])
            sink = float(weights[3]) if len(weights) > 3 else 0.0
            mix = torch.tensor(weights[:3], device=device, dtype=torch.float32)
            scale = mix.repeat_interleave(16).unsqueeze(-1)                            # (48, 1)
            wq, wk = wq * scale, wk * scale
        u = None
        if sink > 0.0:      # extra draws only for heads with a stripe component: the others keep their values
            u = torch.randn(head_dim, generator=g, device=device)
            u = u / u.norm()
            nblk = (nv + SINK_BLOCK - 1) // SINK_BLOCK
            pick = torch.rand(nblk, generator=g, device=device) < (1.0 / SINK_PERIOD)
            on_keys = pick.repeat_interleave(SINK_BLOCK)[:nv].unsqueeze(-1).to(torch.float32)
        for dst, w in ((q, wq), (k, wk)):
            x = 0.5 * torch.randn(nv, head_dim, generator=g, device=device) + gain * (pe @ w)
            if u is not None:
                x += (gain * sink) * u if dst is q else (gain * sink) * u * on_keys
            dst[0, i, v0:v0 + nv] = x.to(dtype)
        v[0, i, v0:v0 + nv] = torch.randn(nv, head_dim, generator=g, device=device).to(dtype)
        if text_tokens:
            for dst in (q, k, v):
                dst[0, i, t0:t0 + text_tokens] = torch.randn(text_tokens, head_dim, generator=g,
                                                             device=device).to(dtype)
    return q, k, v


def make_workload_qkv(name: str, *, seed: int = 1, gain: Optional[float] = None, device="cuda",
                      dtype=torch.bfloat16, head_begin: int = 0, head_end: Optional[int] = None):
    """q, k, v of the named entry of WORKLOADS (its grid, text layout, per-head mixture and positional gain)."""
    cfg = WORKLOADS[name]
    return make_qkv(heads=cfg["heads"], grid=cfg["grid"], head_dim=cfg["head_dim"], text_tokens=cfg["text_tokens"],
                    text_first=cfg["text_first"], seed=seed, gain=cfg.get("gain", 2.0) if gain is None else gain,
                    corr=1.0, axis_mix=cfg.get("axis_mix"), device=device, dtype=dtype, head_begin=head_begin,
                    head_end=head_end)


WORKLOADS = {
    # name: model_type, heads, head_dim, block, grid (T,Hh,Ww), text tokens, text first, top_k, predict_T
    "hunyuan": dict(model_type="hunyuan", heads=24, head_dim=128, block_size=128, grid=(30, 48, 80),
                    text_tokens=256, text_first=False, top_k=300, predict_T=5),
    # per-head mixture: local window / vertical stripes / temporal diagonals, cycling over the heads
    "wan": dict(model_type="wan", heads=40, head_dim=128, block_size=128, grid=(18, 48, 80), text_tokens=0,
                text_first=False, top_k=160, predict_T=10,
                axis_mix=((1.0, 1.0, 1.0), (0.5, 0.5, 0.5, 4.0), (0.2, 1.2, 1.2))),
    # 44,880 video + 224 text tokens at block 64: neither region is a whole number of blocks
    "cogvideox": dict(model_type="cogvideox", heads=48, head_dim=64, block_size=64, grid=(11, 48, 85),
                      text_tokens=224, text_first=True, top_k=100, predict_T=10),
    # the specification's first configuration: 2 heads x 64, block 64, 4096 tokens on a 4 x 32 x 32 grid
    "cfg0": dict(model_type="wan", heads=2, head_dim=64, block_size=64, grid=(4, 32, 32), text_tokens=0,
                 text_first=False, top_k=20, predict_T=5),
    "medium": dict(model_type="hunyuan", heads=8, head_dim=128, block_size=128, grid=(8, 64, 64), text_tokens=256,
                   text_first=False, top_k=80, predict_T=5),
    # a CogVideoX-like case (head_dim 64, block 64, text first) small enough to capture under a profiler
    "medium64": dict(model_type="cogvideox", heads=16, head_dim=64, block_size=64, grid=(4, 64, 64), text_tokens=256,
                     text_first=True, top_k=60, predict_T=5),
    "small": dict(model_type="hunyuan", heads=4, head_dim=128, block_size=128, grid=(8, 32, 32), text_tokens=256,
                  text_first=False, top_k=30, predict_T=5),
}
