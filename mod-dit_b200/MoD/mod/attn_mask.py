"""Adaptive sparse attention state machine on the sm_100a kernels.

Keeps the processor-facing function `SparseAttentionWithMap` and the helper names of the reference's
MoD/mod/attn_mask.py (update_warmup :117-146, compute_block_sparse_map_triton :252-263,
AttentionSparseEngine :266-331, check_bd_values :336-349, choose_topk_lines :351-370,
predict_mask_from_warmup :373-436, generate_mask_from_lines :440-559, SparseAttentionWithMap :567-729).

Differences that are deliberate:
  * every stage runs on this build's kernels; there is no third-party attention kernel, no Triton and
    no CPU path;
  * the block mask is honoured at its native block_size x block_size granularity (the reference's
    third-party sparse kernel coarsens it to 128-row x 64-column tiles);
  * two optional state keys, `score_producer='pooled'` and `selector='cumulative_mass'`, enable the
    mean-pooled map producer and the cumulative-mass selector; their defaults keep reference behaviour;
  * `sparse_type='radial'` runs its static mask (MoD/mod/get_radial_mask.py) through the same sparse
    forward; `sparse_type='spargeattn'` runs the published mean-pooling / top-k method on this library's
    kernels (the third-party package the reference calls is not part of its tree); the 'svg' baseline is not
    part of this build and raises NotImplementedError.
"""
import logging
import math
import weakref
from typing import Dict, List, Optional, Tuple

import torch

from MoD.mod.cuda_lstsq import features_from_solution, solve_lstsq
from MoD.mod.get_radial_mask import get_radial_mask
from MoD.mod.state import is_warmup_complete
from MoD.mod.triton_flash_sparsity import dense_attention_with_lse, flash_attn_with_sparsity_map
from moddit_b200 import _lib
from moddit_b200 import ops as _ops


# ------------------------------------------------------------------------------------------------
# feature extraction
# ------------------------------------------------------------------------------------------------

def extract_attention_features(warmup_state: Dict, S_T: torch.Tensor, blocks_per_frame: int, layer_idx: int = 0,
                               regularization: float = 1, use_cuda: bool = True) -> Dict[str, torch.Tensor]:
    """Fit S_T (H, n, n) onto the line basis; regularisation 1 by default as in the reference (:76-115)."""
    num_heads, n = S_T.shape[0], S_T.shape[1]
    assert S_T.shape == (num_heads, n, n), f"S_T shape mismatch: {S_T.shape} vs ({num_heads}, {n}, {n})"
    return solve_lstsq(warmup_state=warmup_state, S_T=S_T, step=warmup_state['current_steps'], layer_idx=layer_idx,
                       blocks_per_frame=blocks_per_frame, regularization=regularization, use_cuda=use_cuda)


def update_warmup(warmup_state: Dict, step: int, block_sparse_map: torch.Tensor):
    """Append the features of this step's map to the history (:117-146)."""
    if step == warmup_state['warmup_steps'] - 2:
        warmup_state['features_history'] = []
        warmup_state['current_steps'] = step
        warmup_state['prev_full_maps'] = block_sparse_map
    features = extract_attention_features(warmup_state=warmup_state, S_T=block_sparse_map,
                                          blocks_per_frame=warmup_state['blocks_per_frame'],
                                          use_cuda=warmup_state['use_cuda'])
    warmup_state['features_history'].append(features)
    warmup_state['current_steps'] = step + 1
    warmup_state['prev_full_maps'] = block_sparse_map


# ------------------------------------------------------------------------------------------------
# map producers
# ------------------------------------------------------------------------------------------------

def compute_block_sparse_map_triton(query, key, value, warmup_state):
    """Dense output and exact sparsity map (name kept from the reference, :252-263)."""
    return flash_attn_with_sparsity_map(
        query, key, value,
        block_size=warmup_state['block_size'],
        video_token_num=warmup_state['video_token_num'],
        text_token_num=warmup_state['text_token_num'],
        threshold=warmup_state['threshold'],
        model_type=warmup_state['model_type'])


compute_block_sparse_map = compute_block_sparse_map_triton


def _compute_block_sparse_map(query, key, value, *, block_size: int, video_token_num: int, text_token_num: int,
                              threshold: float, model_type: str, q_chunk_blocks: int = 8):
    """Keyword form of the same computation (:152-222, the reference's chunked tensor-expression path; the
    chunk size only bounds its temporaries and is accepted and ignored here: the device path needs none)."""
    del q_chunk_blocks
    return flash_attn_with_sparsity_map(query, key, value, block_size=block_size, video_token_num=video_token_num,
                                        text_token_num=text_token_num, threshold=threshold, model_type=model_type)


def reset_peak_gpu_stats(device: Optional[torch.device] = None):
    """Restart the allocator's peak-memory counters (:41-46)."""
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats(None if device is None else device.index)


def get_cuda_arch_versions() -> List[str]:
    """Compute capability of every visible device as 'sm<major><minor>' (:48-54)."""
    return ["sm%d%d" % torch.cuda.get_device_capability(i) for i in range(torch.cuda.device_count())]


def print_peak_gpu_stats(prefix: str = "", device: Optional[torch.device] = None):
    """Print the peak allocated / reserved device memory in GiB after a synchronize (:56-70)."""
    if not torch.cuda.is_available():
        print(prefix + " GPU not available")
        return
    torch.cuda.synchronize()
    index = None if device is None else device.index
    gib = float(1 << 30)
    print(f"{prefix} peak_alloc={torch.cuda.max_memory_allocated(index) / gib:.3f} GiB, "
          f"peak_reserved={torch.cuda.max_memory_reserved(index) / gib:.3f} GiB")


def compute_pooled_map(query, key, warmup_state, pooled_qk=None) -> torch.Tensor:
    """Mean-pooled stand-in for the sparsity map: (B,H,n,n) float16, same polarity as the exact map.
    `pooled_qk`: block means of query and key computed elsewhere (then query and key are not read)."""
    bs = warmup_state['block_size']
    _, n, off = _geometry(warmup_state, query.shape[2])
    if pooled_qk is not None:
        qbar, kbar = pooled_qk
    else:
        qbar = _ops.pool_blocks(query, bs)
        kbar = _ops.pool_blocks(key, bs)
    return _ops.pooled_map(qbar, kbar, q_block_offset=off, k_block_offset=off, video_blocks=n,
                           scale=query.shape[3] ** -0.5)


def block_geometry(model_type: str, block_size: int, video_token_num: int, text_token_num: int,
                   seq_len: int) -> Tuple[int, int, int]:
    """(blocks in the sequence, video blocks n, index of the first video block) on the block grid that starts
    at token 0.

    For block-aligned shapes these are the reference's floor divisions (:165, :542-557; it accepts nothing
    else).  Shapes it rejects are laid out so that nothing is dropped: the sequence has ceil(seq_len / block_size)
    blocks, the last one short; a block that holds any text token counts as a text block (kept whole, like all
    text rows and columns), so the video blocks are the full-video blocks after (cogvideox) or before (hunyuan)
    the text.  CogVideoX-1.5 at 44,880 video + 224 text tokens and block 64: 705 blocks, 4 text blocks (the fourth
    half text, half video), 701 video blocks of which the last holds 48 tokens."""
    nb = (seq_len + block_size - 1) // block_size
    if model_type == 'wan':
        return nb, nb, 0
    if model_type == 'cogvideox':
        first = min(nb, (text_token_num + block_size - 1) // block_size)
        return nb, nb - first, first
    return nb, min(nb, video_token_num // block_size), 0


def _geometry(warmup_state, seq_len) -> Tuple[int, int, int]:
    return block_geometry(warmup_state['model_type'], warmup_state['block_size'], warmup_state['video_token_num'],
                          warmup_state['text_token_num'], seq_len)


# ------------------------------------------------------------------------------------------------
# sparse engine
# ------------------------------------------------------------------------------------------------

_VALID_KV: Dict[int, Tuple] = {}      # id(mask tensor) -> (weak reference, tensor version, valid length)


def _valid_kv(pre_defined_mask: Optional[torch.Tensor], seq_len: int) -> int:
    """Number of valid (unpadded) keys; reads one row of the caller's mask (a host sync, as :270,281,310).
    The result is remembered per mask tensor object (and its in-place version counter), so a caller that
    passes the same padding mask to every layer and step pays the synchronisation once."""
    if pre_defined_mask is None:
        return seq_len
    key = id(pre_defined_mask)
    hit = _VALID_KV.get(key)
    if hit is not None and hit[0]() is pre_defined_mask and hit[1] == pre_defined_mask._version:
        return hit[2]
    valid = int(pre_defined_mask[0].sum().item())
    if len(_VALID_KV) >= 64:
        _VALID_KV.clear()
    _VALID_KV[key] = (weakref.ref(pre_defined_mask, lambda _ref, key=key: _VALID_KV.pop(key, None)),
                      pre_defined_mask._version, valid)
    return valid


def _engine_lists(mask: torch.Tensor, block_size: int, seq_len: int):
    """(work lists, True when the mask is known on the host to keep every block)."""
    if mask.dim() == 2:
        mask = mask.unsqueeze(0)
    nb = (seq_len + block_size - 1) // block_size
    if mask.shape[-1] != nb or mask.shape[-2] != nb:
        # a mask over the video region only (use_dense passes one): it can only be all-true
        mask = torch.ones(1, nb, nb, device=mask.device, dtype=torch.bool)
        return _ops.tile_lists(mask, block_size, seq_len), True
    return _ops.tile_lists(mask, block_size, seq_len), False


def _events(ready):
    if ready is None:
        return ()
    return tuple(ev for ev in ready if ev is not None) if isinstance(ready, (tuple, list)) else (ready,)


_GROUP_STREAMS: Dict = {}


def _group_streams(device, n: int):
    key = (device.index if device.index is not None else torch.cuda.current_device())
    have = _GROUP_STREAMS.setdefault(key, [])
    while len(have) < n:
        have.append(torch.cuda.Stream(device=device))
    return have[:n]


def _engine_by_head_groups(query, key, value, lists, group_ready, scatter, **fwd_kw):
    """One launch per group of heads, each on a stream of its own behind the event that says the group's rows have
    arrived: the first group computes while the later ones are still on the links.  The lists' order must have been
    made group by group (`tile_lists(..., heads_per_group=...)`).  Returns None with `scatter`, else the output."""
    H = query.shape[1]
    G = len(group_ready)
    hpg = (H + G - 1) // G
    dev = query.device
    main = torch.cuda.current_stream(dev)
    fork = torch.cuda.Event()
    fork.record(main)                      # the lists are complete
    out = None if scatter is not None else torch.empty_like(query)
    npairs = lists.counts.shape[1]
    flat_order = lists.order.view(-1)
    # the launches overlap at their ends: when stages are being timed, one record spans them all, from the first
    # launch (behind its group's arrival) to the end of the last
    timing = _ops.timing_active("moddit_sparse_attn_fwd")
    span_start = None
    with _ops.records_suppressed():
        for g, st in enumerate(_group_streams(dev, G)):
            h0, h1 = g * hpg, min(H, (g + 1) * hpg)
            if h0 >= h1:
                break
            st.wait_event(fork)
            if group_ready[g] is not None:
                st.wait_event(group_ready[g])
            with torch.cuda.stream(st):
                if timing and span_start is None:
                    span_start = torch.cuda.Event(enable_timing=True)
                    span_start.record(st)
                _ops.sparse_attn_fwd(query[:, h0:h1], key[:, h0:h1], value[:, h0:h1], lists.counts[h0:h1],
                                     lists.entries[h0:h1],
                                     order=flat_order[h0 * npairs:h1 * npairs].view(h1 - h0, npairs),
                                     check_status=False, out=None if out is None else out[:, h0:h1],
                                     scatter=None if scatter is None else (scatter[0], scatter[1] + h0), **fwd_kw)
            done = torch.cuda.Event()
            done.record(st)
            main.wait_event(done)
    if span_start is not None:
        span_end = torch.cuda.Event(enable_timing=True)
        span_end.record(main)
        _ops.add_span("moddit_sparse_attn_fwd", span_start, span_end)
    _ops.post_status(dev)
    return out


def AttentionSparseEngine(query, key, value, mask, pre_defined_mask=None, video_token_num=0, block_size=128,
                          _lists=None, _value_ready=None, _scatter=None, _group_ready=None):
    """Block-sparse attention of (B,H,S,D) tensors under a bool block mask (:266-331).

    Video query rows (index < video_token_num) see the keys below the valid length rounded up to 64, text
    rows see exactly the valid keys - the split the reference gets from its two third-party kernels.
    One kernel launch covers both; the result is (B,H,S,D).  When the mask is a stand-in that keeps every
    block (a caller passing a mask of another shape, as the dense steps do), every row sees exactly the valid
    keys, like the reference's dense branch (:268-276).  Whether a full-shape mask happens to be all true is
    not looked up (the reference pays a host synchronisation per call for that): it goes down the sparse
    branch with the 64-rounded border.
    """
    seq_len = query.shape[2]
    query, key = query.contiguous(), key.contiguous()
    all_kept = False
    if _lists is not None:
        lists = _lists
    else:
        lists, all_kept = _engine_lists(mask, block_size, seq_len)
    counts, entries, order = lists.counts, lists.entries, lists.order
    for ev in _events(_value_ready):   # inputs produced on another stream (e.g. still arriving from peers)
        torch.cuda.current_stream(query.device).wait_event(ev)
    value = value.contiguous()
    fwd_kw = {}
    if pre_defined_mask is not None:
        valid = _valid_kv(pre_defined_mask, seq_len)
        border = valid if all_kept else min(seq_len, (valid + 63) // 64 * 64)
        fwd_kw = dict(q_split=video_token_num, kv_len_lo=border, kv_len_hi=valid)
    if _group_ready is not None and len(_group_ready) > 1:
        if query.shape[0] != 1 or lists.counts.shape[0] != query.shape[1]:
            raise ValueError("head groups need a batch of one and one mask per head")
        return _engine_by_head_groups(query, key, value, lists, _group_ready, _scatter, **fwd_kw)
    return _ops.sparse_attn_fwd(query, key, value, counts, entries, order=order, check_status="deferred",
                                scatter=_scatter, **fwd_kw)


# ------------------------------------------------------------------------------------------------
# mask prediction
# ------------------------------------------------------------------------------------------------

def check_bd_values(values: torch.Tensor, mode: List[str], threshold: float = -7.5e-2) -> List[str]:
    """Heads whose last block-diagonal coefficient is <= threshold switch to 'block_diagonal' (:336-349)."""
    codes = _ops.head_modes(values[:, -1], threshold).tolist()
    for i, code in enumerate(codes):
        if mode[i] == 'sparse' and code == _lib.MODE_BLOCK_DIAGONAL:
            mode[i] = 'block_diagonal'
    return mode


def choose_topk_lines(history: List[Dict[str, torch.Tensor]], top_k: int = 10, predict_T: int = None) -> torch.Tensor:
    """Indices (H, k) of the k smallest extrapolated line intensities, verticals first (:351-370)."""
    last, cur = history[-2], history[-1]
    return _ops.select_lines(cur['c'], cur['d'], last['c'], last['d'], top_k, predict_T)


def _mode_codes(mode, device) -> torch.Tensor:
    if torch.is_tensor(mode):
        return mode.to(device=device, dtype=torch.int32)
    return torch.tensor([_lib.MODE_CODE[m] for m in mode], device=device, dtype=torch.int32)


def generate_mask_from_lines(warmup_state: Dict, num_heads: int, n: int, blocks_per_frame: int,
                             selected_lines: torch.Tensor, mode, device: torch.device) -> torch.Tensor:
    """Bool block mask from the selected lines (:440-559); `n` is the sequence length in tokens."""
    model_type = warmup_state.get('model_type')
    if model_type not in _lib.LAYOUT:
        nb = (n + warmup_state['block_size'] - 1) // warmup_state['block_size']
        return torch.ones(num_heads, nb, nb, dtype=torch.bool, device=device)
    total_blocks, video_blocks, first = _geometry(warmup_state, n)
    selected_lines = torch.as_tensor(selected_lines, device=device)
    if selected_lines.dim() == 1:
        selected_lines = selected_lines.unsqueeze(1)
    return _ops.mask_from_lines(selected_lines.long(), _mode_codes(mode, device), n=video_blocks,
                                blocks_per_frame=blocks_per_frame, model_type=model_type,
                                text_blocks=first if model_type == 'cogvideox' else total_blocks - video_blocks,
                                total_blocks=total_blocks)


def predict_mask_from_warmup(warmup_state: Dict, n: int, top_k: int = 10, layer_idx: int = 0) -> Dict:
    """First mask after warm-up: modes from the block-diagonal coefficients, then top-k lines (:373-436)."""
    num_heads = warmup_state['num_heads']
    blocks_per_frame = warmup_state['blocks_per_frame']
    if not is_warmup_complete(warmup_state):
        device = torch.device("cuda")
        nb = _geometry(warmup_state, n)[0]
        return {'mode': ['full'] * num_heads, 'block_diagonal': [False] * num_heads, 'selected_lines': [],
                'mask': torch.ones(num_heads, nb, nb, dtype=torch.bool, device=device)}
    history = warmup_state['features_history']
    device = history[0]['c'].device
    b_d_values = torch.stack([f['b_d'] for f in history], dim=0).to(device).permute(1, 0)
    mode = check_bd_values(b_d_values, threshold=1, mode=['sparse'] * num_heads)
    selected_lines = choose_topk_lines(history, top_k=top_k, predict_T=warmup_state.get('predict_T', None))
    mask = generate_mask_from_lines(warmup_state, num_heads, n, blocks_per_frame, selected_lines, mode, device)
    return {'mode': mode, 'selected_lines': selected_lines, 'mask': mask}


def _store_mask(warmup_state: Dict, mask: torch.Tensor, seq_len: int):
    """Keep the mask and the work lists built from it together, so sparse steps rebuild nothing."""
    warmup_state['mask'] = mask
    full = mask
    bs = warmup_state['block_size']
    nb = (seq_len + bs - 1) // bs
    if mask.shape[-1] != nb:                      # wan: the mask covers the whole (video-only) sequence
        raise ValueError(f"mask of {mask.shape[-1]} blocks does not cover a sequence of {nb} blocks")
    groups = int(warmup_state.get('_head_groups') or 1)
    hpg = (full.shape[0] + groups - 1) // groups if groups > 1 and full.dim() == 3 else None
    warmup_state['_tile_lists'] = (mask, _ops.tile_lists(full, bs, seq_len, heads_per_group=hpg))


def _lists_for(warmup_state: Dict, seq_len: int):
    cached = warmup_state.get('_tile_lists')
    if cached is not None and cached[0] is warmup_state['mask']:
        return cached[1]
    _store_mask(warmup_state, warmup_state['mask'], seq_len)
    return warmup_state['_tile_lists'][1]


def _video_region(warmup_state: Dict, mask: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """(full mask, first video block) so the history merge can index the video region in place."""
    return mask, _geometry(warmup_state, mask.shape[-1] * warmup_state['block_size'])[2]


def _select_and_build(warmup_state: Dict, num_heads: int, seq_len: int, device, dark_map=None):
    if warmup_state.get('selector', 'topk_lines') == 'cumulative_mass':
        keep = _ops.select_mass(dark_map, float(warmup_state.get('mass_threshold', 0.9)))
        return _embed_video_mask(warmup_state, keep, seq_len)
    lines = choose_topk_lines(warmup_state['features_history'], top_k=warmup_state['top_k'],
                              predict_T=warmup_state.get('predict_T', None))
    return generate_mask_from_lines(warmup_state, num_heads, seq_len, warmup_state['blocks_per_frame'], lines,
                                    warmup_state['mode'], device=device)


def _embed_video_mask(warmup_state: Dict, video_mask: torch.Tensor, seq_len: int) -> torch.Tensor:
    if warmup_state['model_type'] == 'wan':
        return video_mask
    nb, n, off = _geometry(warmup_state, seq_len)
    mask = torch.ones(video_mask.shape[0], nb, nb, dtype=torch.bool, device=video_mask.device)
    mask[:, off:off + n, off:off + n] = video_mask
    return mask


# ------------------------------------------------------------------------------------------------
# main entry point
# ------------------------------------------------------------------------------------------------

def SparseAttentionWithMap(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    warmup_state: Dict,
    logger: logging.Logger,
    pre_defined_mask: Optional[torch.Tensor] = None,
    current_step: int = 0,
    layer_idx: int = 0,
    use_dense: bool = False,
    in_test: bool = False,
    **kwargs
) -> Tuple[torch.Tensor, Optional[Dict]]:
    """Adaptive sparse attention of (1, H, S, D) fp16/bf16 tensors (:567-729).

    Optional keyword `value_ready` (a torch.cuda.Event): `value` is produced on another stream and only
    becomes valid once the event has fired; mask prediction, which needs query and key only, starts at
    once and the wait happens right before the attention kernel.
    Optional keywords `pooled_qk` and `qk_ready` (pooled producer only): block means of query and key that
    the caller already holds ((1,H,nb,D) float32 each) and the event after which `query` and `key`
    themselves are valid - a sequence-parallel caller pools its shards before the exchange
    (`moddit_b200.dist.PeerResharder.pool_to_head`), so the mask is predicted while the rows still travel.
    Optional keyword `output_scatter` (from `moddit_b200.dist.PeerResharder.begin_output`): on sparse steps
    the attention kernel stores its rows straight into the peers' sequence-shard buffers and the returned
    output is None; steps that run dense attention ignore it and return the output tensor as usual.
    Optional keyword `head_group_ready` (pooled producer only; a list of G torch.cuda.Events, from
    `PeerResharder.seq_to_head_groups`): query, key and value arrive group of heads by group of heads
    (ceil(H/G) heads each) and event g fires when group g is complete; the block-sparse forward is then launched
    once per group, each launch behind its own event, so the first group computes while the others still travel.
    `warmup_state['_head_groups'] = G` must be set so that the work lists are ordered group by group.

    Steps warmup-2 and warmup-1 collect features (dense output); afterwards every predict_T-th step
    refreshes the map, the features and the mask (dense output) and all other steps run the block-sparse
    forward under the stored mask.  Returns (output (1,H,S,D), mask info) like the reference.
    """
    seq_len = query.size(2)
    num_heads = query.size(1)
    block_size = warmup_state['block_size']
    video_token_num = warmup_state.get('video_token_num', 0)
    # a kernel of an earlier call that gave up a bounded wait is reported here, one call late and without a
    # synchronisation (every attention launch below queues an asynchronous copy of its status words)
    _ops.check_posted_status(query.device)

    if use_dense or warmup_state['sparse_type'] == 'full':
        # 'full' is accepted by create_adaptive_mask_state but has no branch in the reference (:598-729); here it
        # means what its name says: dense attention on every step
        for ev in _events((kwargs.get('value_ready'), kwargs.get('qk_ready'))) + _events(kwargs.get('head_group_ready')):
            torch.cuda.current_stream(query.device).wait_event(ev)     # inputs still arriving on other streams
        query, key, value = query.contiguous(), key.contiguous(), value.contiguous()
        valid = _valid_kv(pre_defined_mask, seq_len)
        output, _ = dense_attention_with_lse(query, key, value, kv_len=valid)
        return output, {'mode': 'warmup', 'mask': None}
    sparse_type = warmup_state['sparse_type']
    if sparse_type == 'svg':
        raise NotImplementedError(f"sparse_type '{sparse_type}' is a third-party baseline that this build does not include")
    if sparse_type == 'spargeattn':
        return _spargeattn_step(query, key, value, warmup_state)
    if sparse_type == 'radial':
        return _radial_step(query, key, value, warmup_state, logger, pre_defined_mask, current_step, layer_idx)

    pooled = warmup_state.get('score_producer', 'replay') == 'pooled'
    warmup_steps = warmup_state['warmup_steps']
    value_ready = kwargs.get('value_ready')
    query, key = query.contiguous(), key.contiguous()

    if pooled:
        return _pooled_step(query, key, value, warmup_state, logger, pre_defined_mask, current_step, layer_idx,
                            value_ready, kwargs.get('output_scatter'), kwargs.get('pooled_qk'),
                            kwargs.get('qk_ready'), kwargs.get('head_group_ready'))
    if kwargs.get('pooled_qk') is not None or kwargs.get('qk_ready') is not None or \
            kwargs.get('head_group_ready') is not None:
        raise ValueError("pooled_qk / qk_ready / head_group_ready need warmup_state['score_producer'] == 'pooled'")
    if value_ready is not None:
        torch.cuda.current_stream(query.device).wait_event(value_ready)
    value = value.contiguous()

    if current_step < warmup_steps:
        if current_step >= warmup_steps - 2:
            output, block_sparse_map = compute_block_sparse_map_triton(query, key, value, warmup_state)
            update_warmup(warmup_state, current_step, block_sparse_map.squeeze(0))
        else:
            output, _ = dense_attention_with_lse(query, key, value, kv_len=_valid_kv(pre_defined_mask, seq_len))
        if current_step == warmup_steps - 1:
            mask_info = predict_mask_from_warmup(warmup_state, seq_len, top_k=warmup_state['top_k'],
                                                 layer_idx=layer_idx)
            warmup_state['mode'] = mask_info['mode']
            mask = mask_info['mask']
            if warmup_state.get('selector', 'topk_lines') == 'cumulative_mass':
                mask = _select_and_build(warmup_state, num_heads, seq_len, query.device,
                                         dark_map=warmup_state['prev_full_maps'])
            _store_mask(warmup_state, mask, seq_len)
            logger.info(f"Layer {layer_idx}, Mask Sparsity: {1 - warmup_state['mask'].float().mean():.3%}")
            _ops.check_health(query.device)         # the two maps the first mask was fitted to are valid
        return output, warmup_state['mask']

    if warmup_state.get('mask', None) is None:
        raise RuntimeError("SparseAttentionWithMap called after warm-up without a mask: the two feature-collection "
                           "steps (warmup_steps-2 and warmup_steps-1) have not run for this layer")
    predict_T = warmup_state['predict_T']
    if (current_step - warmup_steps) % predict_T == predict_T - 1:
        # refresh: dense output + exact map, merged into the history where the current mask kept blocks
        output, current_sparse_map = compute_block_sparse_map_triton(query, key, value, warmup_state)
        current_sparse_map = current_sparse_map.squeeze(0)
        full_mask, off = _video_region(warmup_state, warmup_state['mask'])
        n = current_sparse_map.shape[-1]
        mts, merged = _ops.mts(current_sparse_map, warmup_state['blocks_per_frame'],
                               prev=warmup_state['prev_full_maps'], keep_mask=full_mask, mask_off=off)
        warmup_state['prev_full_maps'] = merged
        X = _ops.solve(mts, n, warmup_state['blocks_per_frame'], 1.0)
        warmup_state['features_history'].append(features_from_solution(X, n))
        warmup_state['features_history'].pop(0)
        next_mask = _select_and_build(warmup_state, num_heads, seq_len, query.device, dark_map=merged)
        _store_mask(warmup_state, next_mask, seq_len)
        _ops.check_health(query.device)             # one synchronising check per refresh (forward and replay map)
    else:
        output = AttentionSparseEngine(query, key, value, warmup_state['mask'], pre_defined_mask=pre_defined_mask,
                                       video_token_num=video_token_num, block_size=block_size,
                                       _lists=_lists_for(warmup_state, seq_len),
                                       _scatter=kwargs.get('output_scatter'))
    return output, {'mask': warmup_state['mask']}


def _radial_step(query, key, value, warmup_state, logger, pre_defined_mask, current_step, layer_idx):
    """`sparse_type='radial'` (:624-630, :713-722): a static mask shared by all heads, built on first use;
    dense attention over all keys during the warm-up steps, the block-sparse forward afterwards."""
    seq_len = query.size(2)
    bs = warmup_state['block_size']
    if bs != 128:
        raise ValueError("the radial mask is built for block_size 128 (the reference never passes another size)")
    query, key, value = query.contiguous(), key.contiguous(), value.contiguous()
    if warmup_state.get('mask', None) is None:
        mask = get_radial_mask(query, warmup_state['video_token_num'], warmup_state['num_frames'],
                               model_type=warmup_state['model_type'])
        nb = (seq_len + bs - 1) // bs
        if mask.shape[-1] != nb:
            raise ValueError(f"mask of {mask.shape[-1]} blocks does not cover a sequence of {nb} blocks")
        warmup_state['mask'] = mask
        # every head shares the mask: one work list serves all heads
        warmup_state['_tile_lists'] = (mask, _ops.tile_lists(mask[:1].contiguous(), bs, seq_len))
        warmup_state['_radial_sparsity'] = 1.0 - float(mask[0].float().mean())
    if current_step < warmup_state['warmup_steps']:
        logger.info(f"Layer {layer_idx}, Mask Sparsity: {warmup_state['_radial_sparsity']:.3%}")
        output, _ = dense_attention_with_lse(query, key, value, kv_len=seq_len)
        return output, {'mode': 'warmup', 'mask': None}
    output = AttentionSparseEngine(query, key, value, warmup_state['mask'], pre_defined_mask=pre_defined_mask,
                                   video_token_num=warmup_state.get('video_token_num', 0), block_size=bs,
                                   _lists=_lists_for(warmup_state, seq_len))
    return output, {'mask': warmup_state['mask']}


def _spargeattn_step(query, key, value, warmup_state):
    """`sparse_type='spargeattn'` (:611-614): the reference hands the whole call to the third-party
    `spas_sage2_attn_meansim_topk_cuda(query, key, value, topk=0.5, is_causal=False)`.  That package is not part
    of the reference tree (an unpinned submodule), so this follows the published method with this library's
    kernels, on every step, over the whole sequence: blocks of query and key are represented by their means,
    every query block keeps the `topk` share (state key `spargeattn_topk`, default 0.5) of key blocks with
    the largest pooled score, and the block-sparse forward runs under that mask.  Blocks whose rows are not
    similar to one another (mean pairwise cosine similarity below state key `spargeattn_sim_threshold`; key
    rows relative to the mean key of the head) are not trusted to their mean: such a query block keeps every
    key block, such a key block is kept by every query block.  The default threshold 0 switches that test off.
    Not taken over: the package's 8-bit quantisation of the products, its 128 x 64 block shape (the mask has
    the state's square block_size) and its skipping of small value products inside the kernel."""
    bs = warmup_state['block_size']
    seq_len = query.size(2)
    query, key, value = query.contiguous(), key.contiguous(), value.contiguous()
    nb = (seq_len + bs - 1) // bs
    qbar, kbar = _ops.pool_blocks(query, bs), _ops.pool_blocks(key, bs)
    dark = _ops.pooled_map(qbar, kbar, q_block_offset=0, k_block_offset=0, video_blocks=nb,
                           scale=float(query.shape[-1]) ** -0.5).squeeze(0)
    threshold = float(warmup_state.get('spargeattn_sim_threshold', 0.0))
    row_full = col_keep = None
    if threshold > 0.0:
        rows = torch.full((nb,), float(bs), device=query.device)
        rows[-1] = float(seq_len - (nb - 1) * bs)
        centre = ((kbar * rows[None, None, :, None]).sum(dim=2) / float(seq_len)).contiguous()   # mean key per head
        row_full = (_ops.block_similarity(query, bs) < threshold).squeeze(0)
        col_keep = (_ops.block_similarity(key, bs, centre) < threshold).squeeze(0)
    count = max(1, min(nb, int(math.ceil(float(warmup_state.get('spargeattn_topk', 0.5)) * nb))))
    mask = _ops.select_topk_blocks(dark, count, row_full, col_keep)
    warmup_state['mask'] = mask
    lists = _ops.tile_lists(mask, bs, seq_len)
    output = _ops.sparse_attn_fwd(query, key, value, lists.counts, lists.entries, order=lists.order,
                                  check_status="deferred")
    return output, {'mode': 'warmup', 'mask': None}


def _pooled_step(query, key, value, warmup_state, logger, pre_defined_mask, current_step, layer_idx,
                 value_ready=None, output_scatter=None, pooled_qk=None, qk_ready=None, head_group_ready=None):
    """Variant with the mean-pooled map producer: the mask is re-predicted on every step from the pooled map
    of that step, so no dense pass is needed after the first feature-collection step."""
    seq_len, num_heads = query.size(2), query.size(1)
    warmup_steps = warmup_state['warmup_steps']
    bs = warmup_state['block_size']

    def wait_value():
        for ev in _events((value_ready, qk_ready)) + _events(head_group_ready):
            torch.cuda.current_stream(query.device).wait_event(ev)

    if current_step < warmup_steps - 2:
        wait_value()
        output, _ = dense_attention_with_lse(query, key, value, kv_len=_valid_kv(pre_defined_mask, seq_len))
        return output, {'mode': 'warmup', 'mask': None}
    if pooled_qk is None:                               # query and key are read by the pooling itself
        for ev in _events(qk_ready) + _events(head_group_ready):
            torch.cuda.current_stream(query.device).wait_event(ev)
    dark = compute_pooled_map(query, key, warmup_state, pooled_qk).squeeze(0)
    n = dark.shape[-1]
    mts, _ = _ops.mts(dark, warmup_state['blocks_per_frame'])
    X = _ops.solve(mts, n, warmup_state['blocks_per_frame'], 1.0)
    feats = features_from_solution(X, n)
    history = warmup_state.get('features_history') or []
    if current_step == warmup_steps - 2 or not history:
        warmup_state['features_history'] = [feats]
        warmup_state['current_steps'] = current_step + 1
        warmup_state['prev_full_maps'] = dark
        wait_value()
        output, _ = dense_attention_with_lse(query, key, value, kv_len=_valid_kv(pre_defined_mask, seq_len))
        return output, {'mode': 'warmup', 'mask': None}
    history.append(feats)
    if len(history) > 2:
        history.pop(0)
    warmup_state['features_history'] = history
    warmup_state['current_steps'] = current_step + 1
    warmup_state['prev_full_maps'] = dark
    warmup_state['mode'] = _ops.head_modes(feats['b_d'], 1.0)     # device-side modes: no host sync per step
    mask = _select_and_build(warmup_state, num_heads, seq_len, query.device, dark_map=dark)
    _store_mask(warmup_state, mask, seq_len)
    output = AttentionSparseEngine(query, key, value, mask, pre_defined_mask=pre_defined_mask,
                                   video_token_num=warmup_state.get('video_token_num', 0), block_size=bs,
                                   _lists=warmup_state['_tile_lists'][1], _value_ready=(value_ready, qk_ready),
                                   _scatter=output_scatter, _group_ready=head_group_ready)
    return output, {'mask': mask}


# ------------------------------------------------------------------------------------------------
# both classifier-free-guidance branches in one call
# ------------------------------------------------------------------------------------------------

_CFG_CONFIG_KEYS = ('model_type', 'num_heads', 'video_token_num', 'text_token_num', 'blocks_per_frame', 'frame_size',
                    'num_frames', 'warmup_steps', 'top_k', 'threshold', 'block_size', 'predict_T', 'sparse_type')
_CFG_OPTION_KEYS = ('score_producer', 'selector', 'mass_threshold', 'spargeattn_topk', 'spargeattn_sim_threshold')


def _cat_heads(parts):
    if any(p is None for p in parts):
        return None
    return torch.cat(list(parts), dim=0)


def _merge_branch_states(states) -> Dict:
    """One state over the heads of all branches (branch b owns heads [b*H, (b+1)*H)), from states that may
    already have run some steps on their own."""
    first = states[0]
    for st in states[1:]:
        for key in _CFG_CONFIG_KEYS + _CFG_OPTION_KEYS:
            if st.get(key) != first.get(key):
                raise ValueError(f"the branches' states differ in '{key}': {first.get(key)!r} vs {st.get(key)!r}")
        if st.get('current_steps') != first.get('current_steps'):
            raise ValueError("the branches' states are at different steps")
    merged = {key: first[key] for key in first if not key.startswith('_')}
    merged['num_heads'] = first['num_heads'] * len(states)
    hist = [st.get('features_history') for st in states]
    if all(h for h in hist):
        merged['features_history'] = [{key: torch.cat([h[i][key] for h in hist], dim=0) for key in hist[0][i]}
                                      for i in range(len(hist[0]))]
    else:
        merged['features_history'] = None if first.get('features_history') is None else []
    merged['prev_full_maps'] = _cat_heads([st.get('prev_full_maps') for st in states])
    merged['mask'] = _cat_heads([st.get('mask') for st in states])
    modes = [st.get('mode') for st in states]
    if all(m is not None for m in modes):
        merged['mode'] = (torch.cat(list(modes)) if torch.is_tensor(modes[0]) else [x for m in modes for x in m])
    else:
        merged.pop('mode', None)
    return merged


def _share_out_branch_states(merged: Dict, states) -> None:
    """Every branch's state dict sees its own heads of the merged state (views: nothing is copied)."""
    nb = len(states)
    H = merged['num_heads'] // nb
    for b, st in enumerate(states):
        lo, hi = b * H, (b + 1) * H
        st['current_steps'] = merged.get('current_steps', st.get('current_steps'))
        hist = merged.get('features_history')
        st['features_history'] = hist if not hist else [{key: f[key][lo:hi] for key in f} for f in hist]
        for key in ('prev_full_maps', 'mask'):
            val = merged.get(key)
            st[key] = None if val is None else (val if val.shape[0] == 1 else val[lo:hi])
        if 'mode' in merged:
            st['mode'] = merged['mode'][lo:hi]
        st.pop('_tile_lists', None)


def SparseAttentionWithMapCFG(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, warmup_states,
                              logger: logging.Logger, pre_defined_mask: Optional[torch.Tensor] = None,
                              current_step: int = 0, layer_idx: int = 0, use_dense: bool = False, **kwargs):
    """Both guidance branches of a layer in one call: `query`, `key`, `value` are (P, H, S, D) with one branch per
    batch item and `warmup_states` holds the P per-branch state dicts.

    The reference's Wan and CogVideoX processors call `SparseAttentionWithMap` once per branch, each with its own
    state (MoD/models/wan/attention_processor.py:144-169, MoD/models/cogvideox/attention_processor.py:185-202).
    Every stage of the path is independent per head, so the branches are run here as P*H heads of one problem:
    one launch of every kernel (the sparse forward walks P*H work lists), one merged state kept under
    `warmup_states[0]['_cfg_merged']`, and after the call every branch's dict shows its own heads of it (mask,
    features, maps) as views.  Output and masks equal those of P separate calls bit for bit.
    Returns (output (P, H, S, D), mask info of the merged state).
    """
    states = list(warmup_states)
    P = len(states)
    if query.dim() != 4 or query.shape[0] != P:
        raise ValueError(f"expected (P={P}, H, S, D) tensors, one batch item per state")
    if pre_defined_mask is not None:
        raise ValueError("the two-branch form has no padded-text rule (no model with guidance branches passes one)")
    H = query.shape[1]
    if H != states[0]['num_heads']:
        raise ValueError(f"{H} heads against a state built for {states[0]['num_heads']}")
    merged = states[0].get('_cfg_merged')
    if merged is None:
        merged = _merge_branch_states(states)
        states[0]['_cfg_merged'] = merged

    def fold(t):
        t = t.contiguous()
        return t.view(1, P * H, t.shape[2], t.shape[3])

    out, info = SparseAttentionWithMap(fold(query), fold(key), fold(value), merged, logger, None, current_step,
                                       layer_idx, use_dense, **kwargs)
    _share_out_branch_states(merged, states)
    return out.view(P, H, out.shape[2], out.shape[3]), info
