"""GPU parity of the exact sparsity-map replay kernel (mirrors the checks of the reference's own test file)."""
import math

import pytest
import torch

from oracle import moddit_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from moddit_b200 import ops as _ops
    return _ops


def _layout(model_type, block_size):
    if model_type == "wan":
        return block_size * 2, block_size * 2, 0
    return block_size * 3, block_size * 2, block_size


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("model_type", ["hunyuan", "cogvideox", "wan"])
@pytest.mark.parametrize("block_size", [64, 128])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_replay_matches_oracle(ops, model_type, block_size, head_dim, dtype, kernel):
    torch.manual_seed(7)
    S, video, text = _layout(model_type, block_size)
    q = torch.randn(2, 2, S, head_dim).to(dtype)
    k = torch.randn(2, 2, S, head_dim).to(dtype)
    lse, scale = orc.replay_lse(q, k)
    n = video // block_size
    off = text if model_type == "cogvideox" else 0
    kw = dict(softmax_scale=scale, log_threshold=math.log(1e-3), q_video_offset=off, k_video_offset=off,
              video_blocks=n, block_size=block_size)
    ref = orc.sparsity_map_replay(q, k, lse, **kw)
    got = ops.replay_map(q.cuda(), k.cuda(), lse.cuda().contiguous(), kernel=kernel, **kw)
    assert ops.replay_status(torch.device("cuda")) == (0, 0, 0, 0)
    assert got.shape == (2, 2, n, n) and got.dtype == torch.float16
    assert torch.all((got >= 0) & (got <= 1))
    # same bound as the reference uses between its two backends (accumulation order moves a few elements)
    assert ((got.cpu().float() - ref.float()).abs() * block_size ** 2).max().item() <= 2.1


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("block_size,n,D", [(128, 9, 128), (64, 9, 64), (64, 16, 128)])
def test_replay_many_tiles_and_odd_block_counts(ops, block_size, n, D, kernel):
    torch.manual_seed(3)
    S = block_size * n + 2 * block_size
    off = block_size
    q = (torch.randn(1, 3, S, D) * 1.5).to(torch.bfloat16)
    k = (torch.randn(1, 3, S, D) * 1.5).to(torch.bfloat16)
    lse, scale = orc.replay_lse(q, k)
    kw = dict(softmax_scale=scale, log_threshold=math.log(2e-3), q_video_offset=off, k_video_offset=off,
              video_blocks=n, block_size=block_size)
    ref = orc.sparsity_map_replay(q, k, lse, **kw)
    got = ops.replay_map(q.cuda(), k.cuda(), lse.cuda(), kernel=kernel, **kw).cpu()
    assert ops.replay_status(torch.device("cuda")) == (0, 0, 0, 0)
    assert ((got.float() - ref.float()).abs() * block_size ** 2).max().item() <= 2.1
    assert 0.05 < got.float().mean().item() < 0.999


@pytest.mark.parametrize("model_type,block_size,head_dim,dtype", [
    ("hunyuan", 128, 128, torch.bfloat16), ("cogvideox", 64, 64, torch.bfloat16), ("wan", 128, 64, torch.float16),
    ("hunyuan", 64, 128, torch.float16)])
def test_the_two_replay_kernels_agree_like_the_reference_backends(model_type, block_size, head_dim, dtype):
    """What tests/test_flash_sparsity.py:61-104 of the reference asserts between its CUDA and its Triton kernel, here
    between the two names those kernels have in this package: same seed, same shapes (B = 2, H = 2), an LSE from
    the scale-then-round convention, at most 2.1 elements of difference per block."""
    from MoD.mod.cuda_flash_sparsity import cuda_sparsity_map
    from MoD.mod.triton_flash_sparsity import _triton_sparsity_map
    torch.manual_seed(7)
    S, video, text = _layout(model_type, block_size)
    q = torch.randn(2, 2, S, head_dim, device="cuda").to(dtype)
    k = torch.randn(2, 2, S, head_dim, device="cuda").to(dtype)
    lse, scale = orc.replay_lse(q.cpu(), k.cpu())
    off = text if model_type == "cogvideox" else 0
    kw = dict(softmax_scale=scale, log_threshold=math.log(1e-3), q_video_offset=off, k_video_offset=off,
              video_blocks=video // block_size, block_size=block_size)
    a = cuda_sparsity_map(q, k, lse.cuda().contiguous(), **kw)
    b = _triton_sparsity_map(q, k, lse.cuda().contiguous(), **kw)
    assert a.shape == b.shape and a.dtype == b.dtype == torch.float16
    assert ((a.float() - b.float()).abs() * block_size ** 2).max().item() <= 2.1
    assert 0.0 < a.float().mean().item() < 1.0


def test_replay_negative_infinite_threshold_gives_zero_map(ops):
    q = torch.randn(1, 1, 128, 64, dtype=torch.float16, device="cuda")
    lse, scale = orc.replay_lse(q.cpu(), q.cpu())
    got = ops.replay_map(q, q, lse.cuda(), softmax_scale=scale, log_threshold=float("-inf"), q_video_offset=0,
                         k_video_offset=0, video_blocks=2, block_size=64)
    assert torch.count_nonzero(got).item() == 0


def test_replay_uses_current_stream(ops):
    q = torch.randn(1, 1, 128, 64, dtype=torch.float16, device="cuda")
    lse, scale = orc.replay_lse(q.cpu(), q.cpu())
    lse = lse.cuda()
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        res = ops.replay_map(q, q, lse, softmax_scale=scale, log_threshold=math.log(1e-3), q_video_offset=0,
                             k_video_offset=0, video_blocks=2, block_size=64)
        marker = res.sum()
    stream.synchronize()
    assert torch.isfinite(marker)


def test_replay_input_errors(ops):
    q = torch.randn(1, 1, 128, 64, dtype=torch.float16, device="cuda")
    lse = torch.zeros(1, 1, 128, device="cuda")
    kw = dict(softmax_scale=0.125, log_threshold=-6.9, q_video_offset=0, k_video_offset=0, video_blocks=2, block_size=64)
    wide = torch.randn(1, 1, 128, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="contiguous"):
        ops.replay_map(wide[..., :64], wide[..., :64], lse, **kw)
    with pytest.raises(RuntimeError, match="float32"):
        ops.replay_map(q, q, lse.half(), **kw)
    with pytest.raises(RuntimeError, match="exceeds sequence length"):
        ops.replay_map(q, q, lse, **{**kw, "video_blocks": 3})
