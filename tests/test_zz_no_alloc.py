"""The allocation-free M^T S entry point (scratch built into the library) against the workspace one.

Some callers cannot give the library a workspace and cannot allocate one either: a plug-in whose host
passes only input and output buffers and forbids device allocation inside the call, or a process whose
framework already owns all device memory.  `moddit_mts_noalloc` serves them.  The file sorts last so
that a run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _grid_map(H, n, bs, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, bs * bs + 1, (H, n, n), generator=g).float() / float(bs * bs)).to(torch.float16)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    from moddit_b200 import _lib, ops
    lib = _lib.lib
    assert lib.moddit_mts_noalloc_max_bytes() == 8 << 20
    # two calls in a row with different sizes: the second must not see anything stale from the first
    for H, n, bpf, seed in ((24, 900, 30, 1), (3, 77, 10, 2)):
        S = _grid_map(H, n, 128, seed).cuda()
        ref, _ = ops.mts(S, bpf)
        out = torch.empty(H, 3 * n, device="cuda", dtype=torch.float32)
        before = torch.cuda.memory_allocated()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = lib.moddit_mts_noalloc(ctypes.c_void_p(S.data_ptr()), H, n, bpf, ctypes.c_void_p(out.data_ptr()), stream)
        assert rc == 0, lib.moddit_last_error_string()
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        # maps on the count/bs^2 grid: line sums are exact, so both entry points agree bit for bit
        assert torch.equal(out[:, :-1], ref[:, :-1])
        assert torch.allclose(out[:, -1], ref[:, -1], rtol=1e-6)
        again = ops.mts_noalloc(S, bpf)
        assert torch.equal(again, out)
        # torch's counter only sees torch's allocator; the driver's own figure must not move either once the first
        # call has loaded the library's module onto the device (that load is when the built-in array is set aside)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.moddit_mts_noalloc(ctypes.c_void_p(S.data_ptr()), H, n, bpf, ctypes.c_void_p(out.data_ptr()), stream)
        torch.cuda.synchronize()
        assert rc == 0 and torch.cuda.mem_get_info()[0] == free_before


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch():
    from moddit_b200 import _lib
    lib = _lib.lib
    H, n = 48, 1024
    assert lib.moddit_mts_workspace_bytes(H, n) > lib.moddit_mts_noalloc_max_bytes()
    S = torch.zeros(1, device="cuda", dtype=torch.float16)
    out = torch.zeros(1, device="cuda", dtype=torch.float32)
    rc = lib.moddit_mts_noalloc(ctypes.c_void_p(S.data_ptr()), H, n, 32, ctypes.c_void_p(out.data_ptr()), None)
    assert rc == -2
    msg = lib.moddit_last_error_string().decode()
    assert "scratch" in msg and "moddit_mts" in msg
