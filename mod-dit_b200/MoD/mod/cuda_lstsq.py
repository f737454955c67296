"""Least-squares fit of a block map onto the diagonal / vertical / block-diagonal basis.

Keeps `solve_lstsq` and its result dictionary from MoD/mod/cuda_lstsq.py:211-270.  M^T S comes from one
fused pass over the map; the shared system is solved through the structured elimination of the C-ABI
library (one data-independent factor per geometry, cached like the reference's Cholesky factor).
"""
import torch

from moddit_b200 import ops as _ops


class _Kernels:
    """Stand-in for the reference's pybind module (MoD/mod/cuda_lstsq_kernel.cu:484-487)."""

    @staticmethod
    def compute_mts(S_T: torch.Tensor, blocks_per_frame: int) -> torch.Tensor:
        return _ops.mts(S_T, int(blocks_per_frame))[0]

    @staticmethod
    def compute_mtm(S_T: torch.Tensor, blocks_per_frame: int, regularization: float) -> torch.Tensor:
        return _ops.mtm(S_T.shape[1], int(blocks_per_frame), float(regularization), S_T.device)


def _load_cuda_extension():
    return _Kernels


def compute_mts_pytorch(S_T: torch.Tensor, blocks_per_frame: int) -> torch.Tensor:
    """M^T S (H, 3n) (name of the reference's tensor-expression twin, :91-139; here the fused device pass,
    which gives the same float32 sums bit for bit on maps of counts / block_size^2)."""
    return _Kernels.compute_mts(S_T, blocks_per_frame)


def compute_mtm_pytorch(S_T: torch.Tensor, blocks_per_frame: int, regularization: float) -> torch.Tensor:
    """M^T M + regularization * I (3n, 3n) (:42-89); only the shape and device of S_T are used."""
    return _Kernels.compute_mtm(S_T, blocks_per_frame, regularization)


def reconstruct_attention_map(features, n, blocks_per_frame=4):
    """The (H, n, n) map that a feature dictionary {'d', 'c', 'b_d'} describes (:271-360)."""
    return _ops.reconstruct_map(features['d'], features['c'], features['b_d'], int(blocks_per_frame))


def features_from_solution(X: torch.Tensor, n: int):
    """Split the raw solution (H, 3n) as MoD/mod/cuda_lstsq.py:257-261 does ('c' is halved)."""
    nd = 2 * n - 1
    return {'d': X[:, :nd], 'c': X[:, nd:nd + n] / 2, 'b_d': X[:, -1]}


def solve_lstsq(warmup_state, S_T, step, blocks_per_frame, layer_idx=0, regularization=1e-5, use_cuda=True):
    """X = (M^T M + reg I)^-1 M^T S for every head of S_T (H, n, n).

    Returns {'d': (H,2n-1) diagonals, 'c': (H,n) verticals / 2, 'b_d': (H,)}; all zeros while
    step <= warmup_steps - 2, as the reference does.  S_T is a float16 map (what both map producers write, as in
    the reference, whose line sums widen it to float32, :231): a float32 S_T is rounded to float16 first.
    """
    num_heads, n = S_T.shape[0], S_T.shape[1]
    if not S_T.is_cuda:
        raise RuntimeError("solve_lstsq needs a CUDA tensor: this build has no CPU path")
    if step > warmup_state['warmup_steps'] - 2:
        mts, _ = _ops.mts(S_T, int(blocks_per_frame))
        X = _ops.solve(mts, n, int(blocks_per_frame), float(regularization))
        return features_from_solution(X, n)
    return {
        'd': torch.zeros((num_heads, 2 * n - 1), device=S_T.device, dtype=torch.float32),
        'c': torch.zeros((num_heads, n), device=S_T.device, dtype=torch.float32),
        'b_d': torch.zeros((num_heads,), device=S_T.device, dtype=torch.float32),
    }
