"""
The allocation-free activation backward, ab200_act_backward_static, against the ordinary entry
point ab200_act_backward.

Some callers of the C ABI cannot allocate device memory: a step running inside a frozen memory
pool, a serving loop that must stay clear of the allocator, or a host program with no allocator of
its own.  For them the library keeps the column-sum scratch in a built-in device array.  This test
calls both entry points through ctypes on the same inputs, twice in a row with different data and
a different shape, and requires identical results: the second call must not see anything the first
left in the shared array.  The file name sorts last so that a run stopping at the first failure has
already run every other test.
"""

import pytest
import torch

from attorch_b200 import _lib

pytestmark = pytest.mark.gpu

DTYPE_ID = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
GELU, NONE = 5, 0


def _run_both(lib, M, N, dtype, act, seed):
    gen = torch.Generator(device='cuda').manual_seed(seed)
    dy = torch.randn(M, N, device='cuda', generator=gen).to(dtype)
    z = torch.randn(M, N, device='cuda', generator=gen).to(dtype)
    stream = torch.cuda.current_stream().cuda_stream
    results = []
    for static in (False, True):
        dz = torch.full((M, N), float('nan'), device='cuda', dtype=dtype)
        db = torch.full((N,), float('nan'), device='cuda', dtype=torch.float32)
        z_ptr = z.data_ptr() if act != NONE else None
        if static:
            rc = lib.ab200_act_backward_static(dy.data_ptr(), z_ptr, dz.data_ptr(), db.data_ptr(), M, N,
                                               N, N, N, DTYPE_ID[dtype], _lib.F32, act, 0.0, stream)
        else:
            nbytes = lib.ab200_act_backward_workspace_bytes(M, N)
            workspace = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
            rc = lib.ab200_act_backward(dy.data_ptr(), z_ptr, dz.data_ptr(), db.data_ptr(), M, N,
                                        N, N, N, DTYPE_ID[dtype], _lib.F32, act, 0.0,
                                        workspace.data_ptr(), nbytes, stream)
        assert rc == 0, _lib.error_string(rc)
        torch.cuda.synchronize()
        results.append((dz, db))
    return results


def test_static_scratch_matches_workspace_entry_point_twice():
    lib = _lib.load()
    # Two calls in a row: the second is smaller and of another type, so stale partial sums of the
    # first call would still sit in the array beyond the region the second one writes.
    for (M, N, dtype, act, seed) in [(1000, 520, torch.bfloat16, GELU, 1), (300, 264, torch.float32, NONE, 2)]:
        (dz_a, db_a), (dz_b, db_b) = _run_both(lib, M, N, dtype, act, seed)
        assert not torch.isnan(dz_b.float()).any() and not torch.isnan(db_b).any()
        assert torch.equal(dz_a, dz_b)
        torch.testing.assert_close(db_b, db_a, rtol=1e-2, atol=1e-2)
        assert torch.equal(db_a, db_b)      # same kernels, same order of additions: same bits


def test_static_scratch_rejects_shapes_beyond_its_capacity():
    lib = _lib.load()
    cap = lib.ab200_act_backward_static_max_floats()
    assert cap == 1 << 20
    N = 4096
    M = (cap // N + 1) * 128                 # one row block too many
    t = torch.empty(16, device='cuda')       # never touched: the shape check comes first
    rc = lib.ab200_act_backward_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), M, N,
                                       N, N, N, _lib.BF16, _lib.F32, GELU, 0.0, None)
    assert rc == -11
    assert 'built-in' in _lib.error_string(rc)
