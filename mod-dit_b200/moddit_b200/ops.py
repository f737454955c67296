"""Tensor-level wrappers over the C ABI: pointer extraction, output allocation, current stream.

Every function here only allocates outputs/workspaces with torch, takes raw device pointers and
calls one `moddit_*` entry point on torch's current stream.  No arithmetic happens in Python and
there is no alternative implementation: CPU tensors are rejected.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import check, lib

_DTYPE = {torch.bfloat16: _lib.MODDIT_BF16, torch.float16: _lib.MODDIT_FP16}

# ---------------------------------------------------------------------------------------------
# optional per-entry-point timing (CUDA events on the launching stream); off by default
# ---------------------------------------------------------------------------------------------
_TIMING = {"on": False, "only": None, "records": [], "launches": 0,
           "nvtx": os.environ.get("MODDIT_NVTX", "0") not in ("", "0")}
# kernels launched by one call of each entry point (for launch accounting in benchmarks)
KERNELS_PER_CALL = {"moddit_pool_blocks": 1, "moddit_pooled_map": 1, "moddit_pooled_map_ws": 3, "moddit_replay_map": 1,
                    "moddit_mts": 2,
                    "moddit_mtm": 1, "moddit_solve": 3, "moddit_select_lines": 1, "moddit_head_modes": 1,
                    "moddit_mask_from_lines": 1, "moddit_select_mass": 1, "moddit_tile_lists": 2,
                    "moddit_sparse_attn_fwd": 1, "moddit_replay_status": 0,
                    "moddit_mts_noalloc": 2, "moddit_copy_rows_dma": 0, "moddit_qkv_prologue": 1}


def stage_timing(enable: bool, only=None) -> None:
    """Turn launch counting and event timing of the entry-point calls on or off and clear the records.
    `only`: names of the entry points to time (all when None); the others are still counted."""
    _TIMING["on"] = bool(enable)
    _TIMING["only"] = None if only is None else frozenset(only)
    _TIMING["records"] = []
    _TIMING["launches"] = 0


def nvtx_ranges(enable: bool) -> None:
    """Wrap every entry-point call in an NVTX range named after it (also switched on by MODDIT_NVTX=1), so a
    timeline shows which launches belong to which stage."""
    _TIMING["nvtx"] = bool(enable)


def stage_records():
    """[(entry point, milliseconds)] since the last `stage_timing(True)`; synchronises the device."""
    torch.cuda.synchronize()
    return [(name, a.elapsed_time(b)) for name, a, b in _TIMING["records"]]


def launches_recorded() -> int:
    return _TIMING["launches"]


def timing_active(name: str) -> bool:
    """Whether calls of entry point `name` are being timed right now."""
    return bool(_TIMING["on"]) and (_TIMING["only"] is None or name in _TIMING["only"])


class records_suppressed:
    """Inside this context entry-point calls are still counted as launches but leave no timing record: for a caller
    that issues several overlapping launches of one kernel on streams of their own and records their common span
    itself (`add_span`), so that the overlap is not counted several times."""

    def __enter__(self):
        self.prev = _TIMING.get("suppress", False)
        _TIMING["suppress"] = True
        return self

    def __exit__(self, *exc):
        _TIMING["suppress"] = self.prev
        return False


def add_span(name: str, start: "torch.cuda.Event", end: "torch.cuda.Event") -> None:
    """A timing record made by the caller (two timing events, possibly recorded on different streams)."""
    if _TIMING["on"]:
        _TIMING["records"].append((name, start, end))


class _timed:
    __slots__ = ("name", "dev", "start")

    def __init__(self, name, dev):
        self.name, self.dev = name, dev

    def __enter__(self):
        self.start = None
        if _TIMING["nvtx"]:
            torch.cuda.nvtx.range_push(self.name)
        if _TIMING["on"] and (_TIMING["only"] is None or self.name in _TIMING["only"]) and not _TIMING.get("suppress"):
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.dev))
        return self

    def __exit__(self, *exc):
        if _TIMING["nvtx"]:
            torch.cuda.nvtx.range_pop()
        if _TIMING["on"]:
            if self.start is not None:
                end = torch.cuda.Event(enable_timing=True)
                end.record(torch.cuda.current_stream(self.dev))
                _TIMING["records"].append((self.name, self.start, end))
            _TIMING["launches"] += KERNELS_PER_CALL.get(self.name, 1)
        return False


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("moddit_b200 ops need CUDA tensors (there is no CPU implementation)")
        if t.device != dev:
            raise ValueError("all tensors must be on the same CUDA device")
    return dev


def _need_contig(**named: torch.Tensor) -> None:
    for name, t in named.items():
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")


def _qkv_dtype(t: torch.Tensor) -> int:
    if t.dtype not in _DTYPE:
        raise TypeError(f"expected float16 or bfloat16 inputs, got {t.dtype}")
    return _DTYPE[t.dtype]


# ---------------------------------------------------------------------------------------------
# pooled map producer
# ---------------------------------------------------------------------------------------------

def pool_blocks(x: torch.Tensor, block_size: int) -> torch.Tensor:
    """(B,H,N,D) bf16/fp16 -> (B,H,ceil(N/bs),D) float32 block means."""
    dev = _need_cuda(x)
    _need_contig(x=x)
    B, H, N, D = x.shape
    nb = (N + block_size - 1) // block_size
    out = torch.empty(B, H, nb, D, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev), _timed("moddit_pool_blocks", dev):
        check(lib.moddit_pool_blocks(_ptr(x), _qkv_dtype(x), B * H, N, D, block_size, _ptr(out), _stream(dev)),
              "moddit_pool_blocks")
    return out


def pool_blocks_shard(x: torch.Tensor, halo_ptr: int, halo_rows: int, halo_capacity: int, block_size: int,
                      n_blocks: int, peer_ptrs, heads_per_peer: int, total_blocks: int, block_base: int) -> None:
    """Pools the blocks of a (1,H,rows,D) sequence shard (preceded by `halo_rows` rows of the halo buffer at
    `halo_ptr`) and stores block i as block `block_base + i` of the head owner's (heads_per_peer,
    total_blocks, D) float32 buffer (`peer_ptrs[h // heads_per_peer]`, device pointers, may be peer memory)."""
    dev = _need_cuda(x)
    _need_contig(x=x)
    B, H, rows, D = x.shape
    if B != 1:
        raise ValueError("pool_blocks_shard: batch must be 1")
    n = len(peer_ptrs)
    table = (ctypes.c_void_p * n)(*peer_ptrs)
    with torch.cuda.device(dev), _timed("moddit_pool_blocks", dev):
        check(lib.moddit_pool_blocks_shard(_ptr(x), ctypes.c_void_p(halo_ptr) if halo_ptr else None, _qkv_dtype(x), H,
                                           rows, halo_rows, halo_capacity, D, block_size, n_blocks, table, n,
                                           heads_per_peer, total_blocks, block_base, _stream(dev)),
              "moddit_pool_blocks_shard")


def qkv_prologue(q_in: Optional[torch.Tensor], k_in: Optional[torch.Tensor], v_in: Optional[torch.Tensor], *,
                 num_heads: int, norm: Optional[str] = None, q_weight: Optional[torch.Tensor] = None,
                 q_bias: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None,
                 k_bias: Optional[torch.Tensor] = None, eps: float = 1e-6,
                 rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None,
                 rope_form: str = "elementwise", rope_range: Optional[Tuple[int, int]] = None,
                 out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None, dst_row0: int = 0,
                 total_tokens: Optional[int] = None, pool_block_size: int = 0,
                 pools: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """Normalisation of q and k, rotary embedding and the token-major -> head-major move in one pass
    (`moddit_qkv_prologue`; the reference does these as separate tensor operations in its processors,
    MoD/models/hunyuan/attention_processor.py:57-106).

    q_in/k_in/v_in: (B, S, H*D) projections (the last dimension contiguous; a slice of a fused projection is
    accepted), any may be None.  norm: None | "rms_head" | "rms_all_heads" | "layer".  rope_cos/rope_sin:
    (rows, D) float32 for the tokens of rope_range (default: all); (rows, D/2), one value per pair, with
    rope_form="pair".  `out`: (q, k, v) buffers (B, H, N_out, D)
    to fill from row `dst_row0` on (allocated with N_out = total_tokens or S when None).  With
    pool_block_size > 0 the block means of the stored q and k are produced as well (`pools` to fill, else
    allocated).  Returns ((q, k, v), (q_pool, k_pool) or None).
    """
    given = [t for t in (q_in, k_in, v_in) if t is not None]
    if not given:
        raise ValueError("qkv_prologue: no input")
    dev = _need_cuda(*given)
    ref = given[0]
    B, S, W = ref.shape
    if W % num_heads:
        raise ValueError(f"inner dimension {W} is not divisible by {num_heads} heads")
    D = W // num_heads
    stride = ref.stride(1)
    for t in given:
        if t.shape != ref.shape or t.dtype != ref.dtype:
            raise ValueError("q_in, k_in and v_in must have one shape and dtype")
        if t.stride(2) != 1 or t.stride(1) != stride or t.stride(0) != S * stride:
            raise ValueError("inputs must be (B, S, H*D) with a contiguous last dimension and one token stride")
    dt = _qkv_dtype(ref)
    for name, p in (("q_weight", q_weight), ("q_bias", q_bias), ("k_weight", k_weight), ("k_bias", k_bias)):
        if p is not None and (p.dtype != ref.dtype or not p.is_contiguous() or p.device != dev):
            raise ValueError(f"{name} must be a contiguous {ref.dtype} tensor on {dev}")
    if (rope_cos is None) != (rope_sin is None):
        raise ValueError("rope_cos and rope_sin go together")
    lo, hi = (0, S) if rope_range is None else rope_range
    if rope_cos is not None:
        width = D // 2 if rope_form == "pair" else D
        for t in (rope_cos, rope_sin):
            if t.dtype != torch.float32 or not t.is_contiguous() or t.shape != (hi - lo, width) or t.device != dev:
                raise ValueError(f"rotary tables must be contiguous float32 ({hi - lo}, {width}) tensors on {dev}")
    N_out = total_tokens if total_tokens is not None else (out[0].shape[2] if out is not None else S)
    if out is None:
        out = tuple(torch.empty(B, num_heads, N_out, D, device=dev, dtype=ref.dtype) for _ in range(3))
    for t in out:
        if t.shape != (B, num_heads, N_out, D) or not t.is_contiguous() or t.dtype != ref.dtype:
            raise ValueError("output buffers must be contiguous (B, H, N_out, D) tensors of the input dtype")
    if pool_block_size > 0 and pools is None:
        nb = (N_out + pool_block_size - 1) // pool_block_size
        pools = tuple(torch.empty(B, num_heads, nb, D, device=dev, dtype=torch.float32) for _ in range(2))
    kind = _lib.NORM_KIND[norm]
    ws_bytes = lib.moddit_qkv_prologue_workspace_bytes(B, S, kind)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8) if ws_bytes else None
    with torch.cuda.device(dev), _timed("moddit_qkv_prologue", dev):
        check(lib.moddit_qkv_prologue(
            _ptr(q_in), _ptr(k_in), _ptr(v_in), dt, B, S, num_heads, D, stride, kind, _ptr(q_weight), _ptr(q_bias),
            _ptr(k_weight), _ptr(k_bias), eps, _ptr(rope_cos), _ptr(rope_sin), _lib.ROPE_FORM[rope_form], lo, hi,
            _ptr(out[0]), _ptr(out[1]), _ptr(out[2]), N_out, dst_row0,
            _ptr(pools[0] if pools is not None and q_in is not None else None),
            _ptr(pools[1] if pools is not None and k_in is not None else None), pool_block_size, _ptr(ws),
            ws_bytes, _stream(dev)), "moddit_qkv_prologue")
    return out, pools


def pooled_map(qbar: torch.Tensor, kbar: torch.Tensor, *, q_block_offset: int, k_block_offset: int,
               video_blocks: int, scale: float, workspace: bool = True) -> torch.Tensor:
    """(B,H,nb,D) float32 block means -> (B,H,n,n) float16 darkness map, 1 - exp(logit - row maximum).

    workspace=True (`moddit_pooled_map_ws`): the means split once, float32 logits tile by tile into a workspace
    (4*B*H*n*n bytes plus the split means), then the row pass; workspace=False (`moddit_pooled_map`): one kernel,
    no workspace, slower.  Both give the same bits."""
    dev = _need_cuda(qbar, kbar)
    _need_contig(qbar=qbar, kbar=kbar)
    if qbar.dtype != torch.float32 or kbar.dtype != torch.float32 or qbar.shape != kbar.shape:
        raise ValueError("qbar and kbar must be float32 tensors of the same shape")
    B, H, nb, D = qbar.shape
    out = torch.empty(B, H, video_blocks, video_blocks, device=dev, dtype=torch.float16)
    if not workspace:
        with torch.cuda.device(dev), _timed("moddit_pooled_map", dev):
            check(lib.moddit_pooled_map(_ptr(qbar), _ptr(kbar), B * H, nb, D, q_block_offset, k_block_offset,
                                        video_blocks, float(scale), _ptr(out), _stream(dev)), "moddit_pooled_map")
        return out
    ws_bytes = int(lib.moddit_pooled_map_workspace_bytes(B * H, video_blocks, D))
    ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev), _timed("moddit_pooled_map_ws", dev):
        check(lib.moddit_pooled_map_ws(_ptr(qbar), _ptr(kbar), B * H, nb, D, q_block_offset, k_block_offset,
                                       video_blocks, float(scale), _ptr(out), _ptr(ws), ws_bytes, _stream(dev)),
              "moddit_pooled_map_ws")
    return out


# ---------------------------------------------------------------------------------------------
# exact replay map
# ---------------------------------------------------------------------------------------------

def replay_map(q: torch.Tensor, k: torch.Tensor, lse: torch.Tensor, *, softmax_scale: float,
               log_threshold: float, q_video_offset: int, k_video_offset: int, video_blocks: int,
               block_size: int, kernel: str = "tcgen05") -> torch.Tensor:
    """Exact sparsity map.  kernel: "tcgen05" (`moddit_replay_map`) or "mma" (`moddit_replay_map_mma`, the second,
    independently written path)."""
    if kernel not in ("tcgen05", "mma"):
        raise ValueError("kernel must be 'tcgen05' or 'mma'")
    dev = _need_cuda(q, k, lse)
    if q.dim() != 4 or k.dim() != 4:
        raise RuntimeError("Q and K must have shape [B, H, S, D]")
    if q.shape != k.shape:
        raise RuntimeError("Q and K shapes must match")
    if lse.dim() != 3 or tuple(lse.shape) != tuple(q.shape[:3]):
        raise RuntimeError("LSE shape must match Q except for head_dim")
    if not (q.is_contiguous() and k.is_contiguous() and lse.is_contiguous()):
        raise RuntimeError("Q, K, and LSE must be contiguous")
    if q.dtype != k.dtype:
        raise RuntimeError("Q and K dtypes must match")
    if q.dtype not in _DTYPE:
        raise RuntimeError("Q and K must be float16 or bfloat16")
    if lse.dtype != torch.float32:
        raise RuntimeError("LSE must be float32")
    B, H, N, D = q.shape
    out = torch.empty(B, H, video_blocks, video_blocks, device=dev, dtype=torch.float16)
    entry = lib.moddit_replay_map if kernel == "tcgen05" else lib.moddit_replay_map_mma
    with torch.cuda.device(dev), _timed("moddit_replay_map", dev):
        rc = entry(_ptr(q), _ptr(k), _ptr(lse), _DTYPE[q.dtype], B * H, N, D, block_size, float(softmax_scale),
                   float(log_threshold), int(q_video_offset), int(k_video_offset), int(video_blocks), _ptr(out),
                   _stream(dev))
    if rc != 0:
        raise RuntimeError("moddit_replay_map: " + lib.moddit_last_error_string().decode())
    return out


def replay_status(device: torch.device) -> Tuple[int, int, int, int]:
    host = (ctypes.c_int32 * 4)()
    with torch.cuda.device(device), _timed("moddit_replay_status", device):
        check(lib.moddit_replay_status(host, _stream(device)), "moddit_replay_status")
    return tuple(int(x) for x in host)


# ---------------------------------------------------------------------------------------------
# least squares
# ---------------------------------------------------------------------------------------------

def mts(S_T: torch.Tensor, blocks_per_frame: int, *, prev: Optional[torch.Tensor] = None,
        keep_mask: Optional[torch.Tensor] = None, mask_off: int = 0
        ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """M^T S of a (H,n,n) float16 map.  With `prev` and `keep_mask` (bool (H,R,R), video region starting at
    block `mask_off`) the history merge `where(keep, S_T, prev)` happens first and is returned too.

    The map is float16 by contract: both producers of this library write float16 maps (the reference's map is
    float16 too and is only widened for the arithmetic, MoD/mod/cuda_lstsq.py:231), and the line sums are then
    exact in float32.  A float32 map is rounded to float16 first - values that are not float16 numbers lose
    their low bits."""
    dev = _need_cuda(S_T)
    if S_T.dtype != torch.float16:
        S_T = S_T.to(torch.float16)
    S_T = S_T.contiguous()
    H, n, _ = S_T.shape
    merged = None
    hs = rs = 0
    if prev is not None:
        if keep_mask is None:
            raise ValueError("prev needs keep_mask")
        prev = prev.to(torch.float16).contiguous()
        keep_mask = keep_mask.contiguous()
        if keep_mask.dtype != torch.bool:
            raise ValueError("keep_mask must be bool")
        hs, rs = keep_mask.stride(0), keep_mask.stride(1)
        merged = torch.empty_like(S_T)
    wsb = lib.moddit_mts_workspace_bytes(H, n)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    out = torch.empty(H, 3 * n, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev), _timed("moddit_mts", dev):
        check(lib.moddit_mts(_ptr(S_T), _ptr(prev), _ptr(keep_mask), hs, rs, mask_off, _ptr(merged), H, n,
                             blocks_per_frame, _ptr(out), _ptr(ws), wsb, _stream(dev)), "moddit_mts")
    return out, merged


def mts_noalloc(S_T: torch.Tensor, blocks_per_frame: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """M^T S through the entry point that allocates nothing: its scratch is an array built into the library.

    For callers that may not allocate device memory inside the call (pass a preallocated `out`); sizes are
    limited by `lib.moddit_mts_noalloc_max_bytes()`.  Calls on one device share the scratch, so calls that
    could overlap on the GPU must be ordered by the caller.
    """
    dev = _need_cuda(S_T)
    if S_T.dtype != torch.float16 or not S_T.is_contiguous():
        raise ValueError("mts_noalloc takes a contiguous float16 (H, n, n) map (converting would allocate)")
    H, n, _ = S_T.shape
    if out is None:
        out = torch.empty(H, 3 * n, device=dev, dtype=torch.float32)
    elif out.dtype != torch.float32 or tuple(out.shape) != (H, 3 * n) or not out.is_contiguous() or out.device != dev:
        raise ValueError("out must be a contiguous float32 (H, 3n) tensor on the map's device")
    with torch.cuda.device(dev), _timed("moddit_mts_noalloc", dev):
        check(lib.moddit_mts_noalloc(_ptr(S_T), H, n, blocks_per_frame, _ptr(out), _stream(dev)),
              "moddit_mts_noalloc")
    return out


def mtm(n: int, blocks_per_frame: int, regularization: float, device) -> torch.Tensor:
    device = torch.device(device)
    out = torch.empty(3 * n, 3 * n, device=device, dtype=torch.float32)
    with torch.cuda.device(device), _timed("moddit_mtm", device):
        check(lib.moddit_mtm(n, blocks_per_frame, float(regularization), _ptr(out), _stream(device)), "moddit_mtm")
    return out


_FACTOR_CACHE: Dict[tuple, torch.Tensor] = {}
_FACTOR_LOCK = threading.Lock()


def reconstruct_map(d: torch.Tensor, c: torch.Tensor, b_d: torch.Tensor, blocks_per_frame: int) -> torch.Tensor:
    """(H,2n-1), (H,n), (H,) float32 line intensities -> (H,n,n) float32 map they describe."""
    dev = _need_cuda(d, c, b_d)
    d, c, b_d = (t.to(torch.float32).contiguous() for t in (d, c, b_d))
    H, n = c.shape
    if d.shape != (H, 2 * n - 1) or b_d.shape != (H,):
        raise ValueError("expected d (H, 2n-1), c (H, n), b_d (H,)")
    out = torch.empty(H, n, n, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev), _timed("moddit_reconstruct_map", dev):
        check(lib.moddit_reconstruct_map(_ptr(d), _ptr(c), _ptr(b_d), H, n, int(blocks_per_frame), _ptr(out),
                                         _stream(dev)), "moddit_reconstruct_map")
    return out


def solve_factor(n: int, blocks_per_frame: int, regularization: float, device) -> torch.Tensor:
    """Inverse of the reduced system for this geometry, computed once per (device, n, bpf, lambda)."""
    device = torch.device(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device(), n,
           int(blocks_per_frame), float(regularization))
    fac = _FACTOR_CACHE.get(key)
    if fac is not None:
        return fac
    with _FACTOR_LOCK:
        fac = _FACTOR_CACHE.get(key)
        if fac is not None:
            return fac
        fb = lib.moddit_solve_factor_bytes(n)
        wb = lib.moddit_solve_prepare_workspace_bytes(n)
        fac = torch.empty(fb, device=device, dtype=torch.uint8)
        ws = torch.empty(wb, device=device, dtype=torch.uint8)
        with torch.cuda.device(device), _timed("moddit_solve_prepare", device):
            check(lib.moddit_solve_prepare(n, blocks_per_frame, float(regularization), _ptr(fac), _ptr(ws), wb,
                                           _stream(device)), "moddit_solve_prepare")
        # other streams may use the factor later: make it globally visible once
        torch.cuda.current_stream(device).synchronize()
        _FACTOR_CACHE[key] = fac
        return fac


def _small_factor(n: int, blocks_per_frame: int, regularization: float, device) -> torch.Tensor:
    """Float32 Cholesky factor of the small system, computed once per (device, n, bpf, lambda)."""
    device = torch.device(device)
    key = ("small", device.index if device.index is not None else torch.cuda.current_device(), n,
           int(blocks_per_frame), float(regularization))
    fac = _FACTOR_CACHE.get(key)
    if fac is not None:
        return fac
    with _FACTOR_LOCK:
        fac = _FACTOR_CACHE.get(key)
        if fac is None:
            fac = torch.empty(lib.moddit_solve_small_factor_bytes(n) // 4, device=device, dtype=torch.float32)
            with torch.cuda.device(device), _timed("moddit_solve_prepare", device):
                check(lib.moddit_solve_small_prepare(n, int(blocks_per_frame), float(regularization), _ptr(fac),
                                                     _stream(device)), "moddit_solve_small_prepare")
            torch.cuda.current_stream(device).synchronize()      # other streams may use the factor later
            _FACTOR_CACHE[key] = fac
        return fac


def solve(mts_: torch.Tensor, n: int, blocks_per_frame: int, regularization: float,
          method: str = "auto") -> torch.Tensor:
    """X (H, 3n) float32 with (M^T M + regularization * I) X = mts.

    method "small": normal equations in shared memory, float32 Cholesky, one warp per head (`moddit_solve_small`;
    n <= `lib.moddit_solve_small_max_n()`); "structured": the float64 structured elimination against a factor
    cached per geometry (`moddit_solve`); "auto": "small" where it fits and regularization >= 0.5, else
    "structured"."""
    dev = _need_cuda(mts_)
    mts_ = mts_.contiguous()
    if mts_.dtype != torch.float32 or mts_.shape[1] != 3 * n:
        raise ValueError("mts must be float32 (H, 3n)")
    if method not in ("auto", "small", "structured"):
        raise ValueError("method must be 'auto', 'small' or 'structured'")
    H = mts_.shape[0]
    # "auto" takes the float32 route only for well-conditioned systems (the regularisation the path uses is 1;
    # with a tiny one the unregularised rank deficiency is a float32 pivot away)
    if method == "small" or (method == "auto" and n <= lib.moddit_solve_small_max_n() and regularization >= 0.5):
        if n > lib.moddit_solve_small_max_n():
            raise ValueError(f"solve: 3n = {3 * n} unknowns exceed the {3 * lib.moddit_solve_small_max_n()} that fit "
                             "shared memory; use method='structured'")
        fac = _small_factor(n, blocks_per_frame, regularization, dev)
        X = torch.empty(H, 3 * n, device=dev, dtype=torch.float32)
        with torch.cuda.device(dev), _timed("moddit_solve", dev):
            check(lib.moddit_solve_small(_ptr(mts_), _ptr(fac), H, n, _ptr(X), _stream(dev)), "moddit_solve_small")
        return X
    fac = solve_factor(n, blocks_per_frame, regularization, dev)
    wb = lib.moddit_solve_workspace_bytes(H, n)
    ws = torch.empty(wb, device=dev, dtype=torch.uint8)
    X = torch.empty(H, 3 * n, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev), _timed("moddit_solve", dev):
        check(lib.moddit_solve(_ptr(mts_), _ptr(fac), H, n, blocks_per_frame, float(regularization), _ptr(X),
                               _ptr(ws), wb, _stream(dev)), "moddit_solve")
    return X


# ---------------------------------------------------------------------------------------------
# selection, masks, work lists
# ---------------------------------------------------------------------------------------------

def select_lines(cur_c, cur_d, last_c, last_d, top_k: int, predict_T: float) -> torch.Tensor:
    dev = _need_cuda(cur_c, cur_d, last_c, last_d)
    ts = [t.to(torch.float32).contiguous() for t in (cur_c, cur_d, last_c, last_d)]
    H, n = ts[0].shape
    if ts[1].shape != (H, 2 * n - 1) or ts[2].shape != (H, n) or ts[3].shape != (H, 2 * n - 1):
        raise ValueError("feature shapes must be c:(H,n) d:(H,2n-1)")
    k = min(int(top_k), 3 * n - 1)
    out = torch.empty(H, k, device=dev, dtype=torch.int64)
    with torch.cuda.device(dev), _timed("moddit_select_lines", dev):
        check(lib.moddit_select_lines(_ptr(ts[0]), _ptr(ts[1]), _ptr(ts[2]), _ptr(ts[3]), H, n, int(top_k),
                                      float(predict_T), _ptr(out), _stream(dev)), "moddit_select_lines")
    return out


def head_modes(b_d: torch.Tensor, threshold: float = 1.0) -> torch.Tensor:
    dev = _need_cuda(b_d)
    b_d = b_d.to(torch.float32).contiguous()
    out = torch.empty(b_d.shape[0], device=dev, dtype=torch.int32)
    with torch.cuda.device(dev), _timed("moddit_head_modes", dev):
        check(lib.moddit_head_modes(_ptr(b_d), b_d.shape[0], float(threshold), _ptr(out), _stream(dev)),
              "moddit_head_modes")
    return out


def mask_from_lines(selected: torch.Tensor, modes: torch.Tensor, *, n: int, blocks_per_frame: int,
                    model_type: str, text_blocks: int, total_blocks: int) -> torch.Tensor:
    dev = _need_cuda(selected, modes)
    if model_type not in _lib.LAYOUT:
        raise ValueError(f"Unknown model_type: {model_type}, expected 'wan', 'hunyuan', or 'cogvideox'")
    selected = selected.to(torch.int64).contiguous()
    modes = modes.to(torch.int32).contiguous()
    H, k = selected.shape
    nbt = n if model_type == "wan" else total_blocks
    mask = torch.empty(H, nbt, nbt, device=dev, dtype=torch.bool)
    with torch.cuda.device(dev), _timed("moddit_mask_from_lines", dev):
        check(lib.moddit_mask_from_lines(_ptr(selected), k, _ptr(modes), H, n, blocks_per_frame,
                                         _lib.LAYOUT[model_type], text_blocks, nbt, _ptr(mask), _stream(dev)),
              "moddit_mask_from_lines")
    return mask


def radial_mask(model_type: str, video_token_num: int, num_frames: int, seq_len: int, device: torch.device,
                block_size: int = 128, decay_factor: float = 0.2) -> torch.Tensor:
    """(seq_len//block_size, seq_len//block_size) bool: the static radial block mask (one head)."""
    if model_type not in ("hunyuan", "wan"):
        raise ValueError(f"Unknown model type: {model_type}")
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("moddit_b200 runs on CUDA devices only (no CPU fallback)")
    nb = seq_len // block_size
    mask = torch.empty(nb, nb, device=device, dtype=torch.bool)
    with torch.cuda.device(device), _timed("moddit_radial_mask", device):
        check(lib.moddit_radial_mask(_lib.LAYOUT[model_type], int(video_token_num), int(num_frames), int(seq_len),
                                     int(block_size), float(decay_factor), _ptr(mask), _stream(device)),
              "moddit_radial_mask")
    return mask


def select_mass(dark_map: torch.Tensor, tau: float) -> torch.Tensor:
    dev = _need_cuda(dark_map)
    dark_map = dark_map.to(torch.float16).contiguous()
    H, n, _ = dark_map.shape
    keep = torch.empty(H, n, n, device=dev, dtype=torch.bool)
    with torch.cuda.device(dev), _timed("moddit_select_mass", dev):
        check(lib.moddit_select_mass(_ptr(dark_map), H, n, float(tau), _ptr(keep), _stream(dev)),
              "moddit_select_mass")
    return keep


def block_similarity(x: torch.Tensor, block_size: int, center: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(B,H,N,D) bf16/fp16 -> (B,H,ceil(N/bs)) float32: mean pairwise cosine similarity of the rows of every
    block, after subtracting `center` ((B,H,D) float32) from the rows when given."""
    dev = _need_cuda(x)
    _need_contig(x=x)
    B, H, N, D = x.shape
    if center is not None:
        if center.shape != (B, H, D) or center.dtype != torch.float32 or not center.is_contiguous():
            raise ValueError("center must be a contiguous (B, H, D) float32 tensor")
    out = torch.empty(B, H, (N + block_size - 1) // block_size, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev), _timed("moddit_block_similarity", dev):
        check(lib.moddit_block_similarity(_ptr(x), _qkv_dtype(x), B * H, N, D, block_size, _ptr(center), _ptr(out),
                                          _stream(dev)), "moddit_block_similarity")
    return out


def select_topk_blocks(dark_map: torch.Tensor, count: int, row_full: Optional[torch.Tensor] = None,
                       col_keep: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(H,n,n) float16 map (0 = brightest) -> (H,n,n) bool: per row the `count` brightest blocks, plus whole
    rows where row_full (H,n) and whole columns where col_keep (H,n) are set."""
    dev = _need_cuda(dark_map)
    dark_map = dark_map.to(torch.float16).contiguous()
    H, n, _ = dark_map.shape
    flags = []
    for f in (row_full, col_keep):
        if f is not None:
            if f.shape != (H, n) or f.device != dev:
                raise ValueError("row_full / col_keep must be (H, n) tensors on the map's device")
            f = f.to(torch.bool).contiguous()
        flags.append(f)
    keep = torch.empty(H, n, n, device=dev, dtype=torch.bool)
    with torch.cuda.device(dev), _timed("moddit_select_topk_blocks", dev):
        check(lib.moddit_select_topk_blocks(_ptr(dark_map), H, n, int(count), _ptr(flags[0]), _ptr(flags[1]), _ptr(keep),
                                            _stream(dev)), "moddit_select_topk_blocks")
    return keep


class TileLists(tuple):
    """(counts, entries, order) produced by `tile_lists`; unpacks like the 2-tuple (counts, entries)."""

    def __new__(cls, counts, entries, order):
        obj = super().__new__(cls, (counts, entries))
        obj.counts, obj.entries, obj.order = counts, entries, order
        return obj

    def __getnewargs__(self):          # lets a state dict that holds work lists be pickled / torch.save'd
        return self.counts, self.entries, self.order


def tile_lists(mask: torch.Tensor, block_size: int, n_tokens: int, kv_block_limit: Optional[int] = None,
               heads_per_group: Optional[int] = None) -> TileLists:
    """Work lists of the sparse forward for a bool (H, nbq, nbk) block mask, plus the start order of the
    (head, query-tile pair) work items (long lists first).  With `heads_per_group` the order is made group by
    group of that many heads (`moddit_order_pairs`), for one launch per group over slices of the lists."""
    dev = _need_cuda(mask)
    if mask.dtype != torch.bool or mask.dim() != 3:
        raise ValueError("mask must be a bool (H, nbq, nbk) tensor")
    mask = mask.contiguous()
    Hm, nbq, nbk = mask.shape
    ntq = (n_tokens + 127) // 128
    npairs = (ntq + 1) // 2
    counts = torch.empty(Hm, npairs, device=dev, dtype=torch.int32)
    entries = torch.empty(Hm, npairs, ntq, device=dev, dtype=torch.int32)
    order = torch.empty(Hm, npairs, device=dev, dtype=torch.int32)
    lim = nbk if kv_block_limit is None else int(kv_block_limit)
    grouped = heads_per_group is not None and 0 < int(heads_per_group) < Hm
    with torch.cuda.device(dev), _timed("moddit_tile_lists", dev):
        check(lib.moddit_tile_lists(_ptr(mask), Hm, nbq, nbk, block_size, n_tokens, lim, _ptr(counts),
                                    _ptr(entries), None if grouped else _ptr(order), _stream(dev)), "moddit_tile_lists")
        if grouped:
            check(lib.moddit_order_pairs(_ptr(counts), Hm, npairs, int(heads_per_group), _ptr(order), _stream(dev)),
                  "moddit_order_pairs")
    return TileLists(counts, entries, order)


def copy_rows(src_ptr: int, dst_ptr: int, src_pitch: int, dst_pitch: int, width_bytes: int, rows: int,
              device: torch.device) -> None:
    """Raw strided row copy on `device`'s current stream; `dst_ptr` may point into a peer GPU's mapped buffer."""
    with torch.cuda.device(device), _timed("moddit_copy_rows", device):
        check(lib.moddit_copy_rows(ctypes.c_void_p(src_ptr), ctypes.c_void_p(dst_ptr), src_pitch, dst_pitch,
                                   width_bytes, rows, _stream(device)), "moddit_copy_rows")


def copy_rows_dma(src_ptr: int, dst_ptr: int, src_pitch: int, dst_pitch: int, width_bytes: int, rows: int,
                  device: torch.device) -> None:
    """`copy_rows` on the copy engines (no kernel launch, hence not counted as one)."""
    with torch.cuda.device(device), _timed("moddit_copy_rows_dma", device):
        check(lib.moddit_copy_rows_dma(ctypes.c_void_p(src_ptr), ctypes.c_void_p(dst_ptr), src_pitch, dst_pitch,
                                       width_bytes, rows, _stream(device)), "moddit_copy_rows_dma")


def copy_rows_multi(src_ptrs, dst_ptrs, src_pitch: int, dst_pitch: int, width_bytes: int, rows: int,
                    device: torch.device) -> None:
    """`copy_rows` for several (source, destination) pointer pairs in one launch."""
    n = len(src_ptrs)
    src = (ctypes.c_void_p * n)(*src_ptrs)
    dst = (ctypes.c_void_p * n)(*dst_ptrs)
    with torch.cuda.device(device), _timed("moddit_copy_rows", device):
        check(lib.moddit_copy_rows_multi(src, dst, n, src_pitch, dst_pitch, width_bytes, rows, _stream(device)),
              "moddit_copy_rows_multi")


def copy_rows_narrow(src_ptrs, dst_ptrs, src_pitch: int, dst_pitch: int, width_bytes: int, rows: int,
                     device: torch.device, max_ctas: int = 48) -> None:
    """`copy_rows_multi` on at most `max_ctas` CTAs (an exchange that runs beside other kernels)."""
    n = len(src_ptrs)
    src = (ctypes.c_void_p * n)(*src_ptrs)
    dst = (ctypes.c_void_p * n)(*dst_ptrs)
    with torch.cuda.device(device), _timed("moddit_copy_rows", device):
        check(lib.moddit_copy_rows_narrow(src, dst, n, src_pitch, dst_pitch, width_bytes, rows, int(max_ctas),
                                          _stream(device)), "moddit_copy_rows_narrow")


# ---------------------------------------------------------------------------------------------
# sparse forward
# ---------------------------------------------------------------------------------------------

_STATUS: Dict[int, torch.Tensor] = {}
_POSTED: Dict[int, list] = {}        # device index -> [pinned int32[4] copy of the status words, event or None]


def _status_words(dev: torch.device) -> torch.Tensor:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _STATUS.get(idx)
    if st is None:
        st = torch.zeros(4, device=dev, dtype=torch.int32)
        _STATUS[idx] = st
    return st


def _status_error(vals) -> "_lib.ModditError":
    return _lib.ModditError(
        f"sparse_attn_fwd: a bounded wait expired inside the kernel (code={vals[0]} block={vals[1]} "
        f"role={vals[2]} position={vals[3]}); the output is invalid")


def raise_on_status(device) -> None:
    """Synchronising check of the sparse forward's status words on `device`."""
    device = torch.device(device)
    st = _status_words(device)
    vals = st.tolist()
    if vals[0] != 0:
        st.zero_()
        raise _status_error(vals)


def post_status(device) -> None:
    """Queues a copy of the status words into pinned host memory behind the work already on the current stream
    and records an event after it.  Costs no synchronisation; `check_posted_status` looks at the copy later."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    slot = _POSTED.get(idx)
    if slot is None:
        slot = [torch.zeros(4, dtype=torch.int32).pin_memory(), None]
        _POSTED[idx] = slot
    if slot[1] is not None and not slot[1].query():
        return                                   # the previous copy has not landed yet: it reports the same words
    slot[0].copy_(_status_words(device), non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(device))
    slot[1] = ev


def check_posted_status(device) -> None:
    """Looks at the last posted copy of the status words if it has arrived (never waits): raises ModditError when
    a kernel launched before that copy gave up a bounded wait.  Called at the start of every attention-layer
    call, so a fault surfaces one call later without a synchronisation per step."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    slot = _POSTED.get(idx)
    if slot is None or slot[1] is None or not slot[1].query():
        return
    slot[1] = None
    vals = slot[0].tolist()
    if vals[0] != 0:
        _status_words(device).zero_()
        raise _status_error(vals)


def check_health(device) -> None:
    """Synchronising check of every kernel status this library keeps on `device` (sparse/dense forward and
    replay map): for the end of a denoising step or of a run."""
    device = torch.device(device)
    raise_on_status(device)
    vals = replay_status(device)
    if vals[0] != 0:
        raise _lib.ModditError(
            f"replay_map: a bounded wait expired inside the kernel (code={vals[0]} block={vals[1]} role={vals[2]} "
            f"position={vals[3]}); the sparsity maps written since the last check are invalid")


def _after_launch(dev, check_status) -> None:
    if check_status == "deferred":
        post_status(dev)
    elif check_status:
        raise_on_status(dev)


def sparse_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, counts: torch.Tensor,
                    entries: torch.Tensor, *, order: Optional[torch.Tensor] = None,
                    softmax_scale: Optional[float] = None,
                    q_split: Optional[int] = None, kv_len_lo: Optional[int] = None,
                    kv_len_hi: Optional[int] = None, return_lse: bool = False, check_status=True,
                    out: Optional[torch.Tensor] = None, scatter=None):
    """Block-sparse attention forward of (B,H,N,D) tensors over the work lists from `tile_lists`.

    check_status: True reads the kernel's status words after the launch (synchronises); "deferred" queues an
    asynchronous copy of them (`post_status`) for a later `check_posted_status`; False does neither."""
    dev = _need_cuda(q, k, v, counts, entries)
    _need_contig(q=q, k=k, v=v, counts=counts, entries=entries)
    if q.shape != k.shape or q.shape != v.shape or q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("query, key, and value must have identical shapes and dtypes")
    B, H, N, D = q.shape
    Hm = counts.shape[0]
    ntq = (N + 127) // 128
    if counts.dtype != torch.int32 or entries.dtype != torch.int32 or \
            tuple(counts.shape) != (Hm, (ntq + 1) // 2) or tuple(entries.shape) != (Hm, (ntq + 1) // 2, ntq):
        raise ValueError("counts/entries do not match the sequence length (see tile_lists)")
    if order is not None and (order.dtype != torch.int32 or tuple(order.shape) != tuple(counts.shape)
                              or not order.is_contiguous() or order.device != dev):
        raise ValueError("order must be the contiguous int32 (Hm, npairs) tensor from tile_lists")
    scale = float(D ** -0.5 if softmax_scale is None else softmax_scale)
    lse = torch.empty(B, H, N, device=dev, dtype=torch.float32) if return_lse else None
    st = _status_words(dev)
    if scatter is not None:
        # scatter = (peer buffer pointers, head_base): output rows go straight into the peers' buffers
        peer_ptrs, head_base = scatter
        table = (ctypes.c_void_p * len(peer_ptrs))(*peer_ptrs)
        with torch.cuda.device(dev), _timed("moddit_sparse_attn_fwd", dev):
            check(lib.moddit_sparse_attn_fwd_scatter(
                _ptr(q), _ptr(k), _ptr(v), _qkv_dtype(q), B * H, N, D, _ptr(counts), _ptr(entries), _ptr(order), Hm,
                scale, N if q_split is None else int(q_split), N if kv_len_lo is None else int(kv_len_lo),
                N if kv_len_hi is None else int(kv_len_hi), table, len(peer_ptrs), int(head_base), _ptr(lse),
                _ptr(st), _stream(dev)), "moddit_sparse_attn_fwd_scatter")
        _after_launch(dev, check_status)
        return (None, lse) if return_lse else None
    if out is None:
        out = torch.empty_like(q)
    with torch.cuda.device(dev), _timed("moddit_sparse_attn_fwd", dev):
        check(lib.moddit_sparse_attn_fwd(_ptr(q), _ptr(k), _ptr(v), _qkv_dtype(q), B * H, N, D, _ptr(counts),
                                         _ptr(entries), _ptr(order), Hm, scale, N if q_split is None else int(q_split),
                                         N if kv_len_lo is None else int(kv_len_lo),
                                         N if kv_len_hi is None else int(kv_len_hi), _ptr(out), _ptr(lse),
                                         _ptr(st), _stream(dev)), "moddit_sparse_attn_fwd")
    _after_launch(dev, check_status)
    return (out, lse) if return_lse else out
