#!/usr/bin/env python3
"""Times the exact sparsity-map replay and the full refresh step (dense forward + replay) on one GPU.

Same command line and output format as the reference's benchmarks/benchmark_flash_sparsity.py (median / p20 /
p80 of CUDA-event timings), plus the tensor throughput each figure corresponds to.  The log-sum-exp for the
replay-only rows comes from this build's own dense forward.
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from MoD.mod.cuda_flash_sparsity import cuda_backend_supported, cuda_sparsity_map  # noqa: E402
from MoD.mod.triton_flash_sparsity import dense_attention_with_lse, flash_attn_with_sparsity_map  # noqa: E402


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--heads", type=int, default=24)
    p.add_argument("--sequence", type=int, default=4096)
    p.add_argument("--head-dim", type=int, choices=(64, 128), default=128)
    p.add_argument("--block-size", type=int, choices=(64, 128), default=128)
    p.add_argument("--text-tokens", type=int, default=128)
    p.add_argument("--model-type", choices=("hunyuan", "cogvideox", "wan"), default="hunyuan")
    p.add_argument("--threshold", type=float, default=1e-4)
    p.add_argument("--dtype", choices=("fp16", "bf16"), default="fp16")
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--repetitions", type=int, default=100)
    return p.parse_args()


def quantile(values, q):
    values = sorted(values)
    pos = (len(values) - 1) * q
    lo = int(pos)
    hi = min(lo + 1, len(values) - 1)
    return values[lo] * (1.0 - (pos - lo)) + values[hi] * (pos - lo)


def measure(op, warmup, repetitions):
    for _ in range(warmup):
        op()
    torch.cuda.synchronize()
    samples = []
    for _ in range(repetitions):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        op()
        b.record()
        b.synchronize()
        samples.append(a.elapsed_time(b))
    return {"p20": quantile(samples, 0.2), "median": quantile(samples, 0.5), "p80": quantile(samples, 0.8)}


def show(label, res, flops):
    print(f"{label:28s} median={res['median']:8.3f} ms  p20={res['p20']:8.3f}  p80={res['p80']:8.3f}  "
          f"{flops / res['median'] / 1e9:8.1f} TFLOP/s")


def main():
    a = parse_args()
    if not torch.cuda.is_available() or not cuda_backend_supported():
        raise SystemExit("an sm_100 CUDA device is required")
    dtype = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    video = a.sequence if a.model_type == "wan" else a.sequence - a.text_tokens
    if video % a.block_size:
        raise SystemExit("video token count must be divisible by block size")
    off = a.text_tokens if a.model_type == "cogvideox" else 0
    n = video // a.block_size
    scale = a.head_dim ** -0.5
    log_thr = math.log(a.threshold) if a.threshold > 0 else float("-inf")
    torch.manual_seed(123)
    q = torch.randn(a.batch, a.heads, a.sequence, a.head_dim, device="cuda", dtype=dtype)
    k, v = torch.randn_like(q), torch.randn_like(q)
    _, lse = dense_attention_with_lse(q, k, v, scale)
    kw = dict(softmax_scale=scale, log_threshold=log_thr, q_video_offset=off, k_video_offset=off, video_blocks=n,
              block_size=a.block_size)
    bh = a.batch * a.heads
    replay_flops = 2.0 * video * video * a.head_dim * bh
    dense_flops = 4.0 * a.sequence * a.sequence * a.head_dim * bh
    show("replay map (tcgen05)", measure(lambda: cuda_sparsity_map(q, k, lse, **kw), a.warmup, a.repetitions),
         replay_flops)
    show("dense forward + LSE", measure(lambda: dense_attention_with_lse(q, k, v, scale), a.warmup, a.repetitions),
         dense_flops)
    show("forward + replay (public API)", measure(
        lambda: flash_attn_with_sparsity_map(q, k, v, a.threshold, a.block_size, model_type=a.model_type,
                                             video_token_num=0 if a.model_type == "wan" else video,
                                             text_token_num=a.text_tokens), a.warmup, a.repetitions),
         replay_flops + dense_flops)


if __name__ == "__main__":
    main()
