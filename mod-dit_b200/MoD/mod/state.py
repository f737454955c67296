"""Per-layer state of the adaptive sparse attention: same keys as the reference's MoD/mod/state.py:3-72.

Two optional keys select the variants that only this build has; their defaults keep the reference
behaviour:
    score_producer : 'replay' (exact sparsity map, refresh steps only) | 'pooled' (mean-pooled map, every step)
    selector       : 'topk_lines' | 'cumulative_mass' (uses `mass_threshold`)
"""
from typing import Dict

_SPARSE_TYPES = {'full', 'mod-dit', 'radial', 'svg', 'spargeattn'}


def init_warmup_state() -> Dict:
    """Empty algorithm state (MoD/mod/state.py:3-22)."""
    return {
        'features_history': None,
        'current_steps': 0,
        'prev_full_maps': None,
        'prediction_features': {},
        'mask': None,
        'sparse_id': None,
    }


def create_adaptive_mask_state(
    model_type: str,
    num_heads: int,
    video_token_num: int,
    text_token_num: int,
    tokens_per_frame: int,
    num_frames: int,
    warmup_steps: int = 12,
    top_k: int = 10,
    predict_T: int = 5,
    threshold: float = 1.5e-4,
    block_size: int = 128,
    use_cuda: bool = True,
    sparse_type: str = 'mod-dit',
) -> Dict:
    """Configuration plus empty algorithm state for one attention layer (MoD/mod/state.py:24-68)."""
    state = init_warmup_state()
    state.update(
        model_type=model_type,
        num_heads=num_heads,
        video_token_num=video_token_num,
        text_token_num=text_token_num,
        blocks_per_frame=tokens_per_frame // block_size,
        frame_size=tokens_per_frame,
        num_frames=num_frames,
        warmup_steps=warmup_steps,
        top_k=top_k,
        threshold=float(threshold),
        block_size=block_size,
        predict_T=predict_T,
        use_cuda=use_cuda,
    )
    if sparse_type not in _SPARSE_TYPES:
        raise ValueError(f"{sparse_type} not support , only support [full mod-dit, radial, svg, spargeattn]")
    state['sparse_type'] = sparse_type
    return state


def is_warmup_complete(warmup_state: Dict) -> bool:
    """True once `current_steps` reached `warmup_steps` (MoD/mod/state.py:70-72)."""
    return warmup_state['current_steps'] >= warmup_state['warmup_steps']
