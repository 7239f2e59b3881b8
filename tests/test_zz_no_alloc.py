"""The allocation-free submanifold rulebook entry point (ssc_rulebook_subm_static).

Some users of the library cannot allocate device memory at call time: a plugin whose host
application owns the whole device pool, a service that freezes its memory after start-up so
that no request can fail on an allocation, a build without an allocator.  For them the
library carries its scratch in a fixed internal array.  This test calls the entry point
through the C ABI (ctypes, raw pointers) and requires bit-identical results to the regular
entry point that works in caller-provided scratch, on two different inputs in a row, because
the internal array is shared by all calls and keeps the previous call's contents.

The file name makes pytest collect it last, so a run that stops at the first failure has
already executed every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(L, ext, ind_np, batch, shape, ksize, dilation, dev):
    ind = torch.from_numpy(np.ascontiguousarray(ind_np)).to(dev).contiguous()
    n = ind.shape[0]
    K = ksize[0] * ksize[1] * ksize[2]
    I3 = ctypes.c_int * 3
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    res = []
    for static in (False, True):
        # outputs belong to the caller in both variants; poison them so stale data would show
        nbr = torch.full((K, n), -7, dtype=torch.int32, device=dev)
        pairs = torch.full((K, 2, n), -7, dtype=torch.int32, device=dev)
        num = torch.full((K,), -7, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())
        if static:
            rc = L.ssc_rulebook_subm_static(ptr(ind), n, batch, I3(*shape), I3(*ksize), I3(*dilation), ptr(nbr),
                                            ptr(pairs), ptr(num), ptr(status), stream)
        else:
            nbytes = L.ssc_rulebook_scratch_bytes(n, batch, I3(*shape), I3(*shape), K)
            scratch = torch.empty(int(nbytes), dtype=torch.uint8, device=dev)
            rc = L.ssc_rulebook_subm(ptr(ind), n, batch, I3(*shape), I3(*ksize), I3(*dilation), ptr(nbr), ptr(pairs),
                                     ptr(num), ptr(status), ptr(scratch), scratch.numel(), stream)
        assert rc == 0, L.ssc_last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0, ("static" if static else "regular", n, batch, shape, ksize)
        res.append((nbr.cpu().numpy(), pairs.cpu().numpy(), num.cpu().numpy()))
    return res


def test_static_scratch_rulebook_matches_regular_entry_point(cuda):
    from ss_conv import _ext
    from ss_conv.utils import synthetic as S
    L = _ext.lib()
    first = S.surface_voxels(range(4), 32, 4096, base_seed=11)          # ~7k voxels, k = 3
    second = S.bernoulli_voxels(range(2), 24, 0.1, base_seed=5)          # different size, k = 5
    for ind, batch, shape, ksize in ((first, 4, [32] * 3, [3] * 3), (second, 2, [24] * 3, [5] * 3)):
        (nbr_a, pairs_a, num_a), (nbr_b, pairs_b, num_b) = _both(L, _ext, ind, batch, shape, ksize, [1, 1, 1], cuda)
        assert np.array_equal(num_a, num_b)
        assert np.array_equal(nbr_a, nbr_b)          # integer work: bit-exact
        assert np.array_equal(pairs_a, pairs_b)
        assert num_a[len(num_a) // 2] == ind.shape[0]    # centre offset pairs every voxel with itself
    # exactly at the documented limit: 65 536 active voxels (a 16 x 64 x 64 slab, fully occupied)
    full = np.stack(np.meshgrid(np.arange(16), np.arange(64), np.arange(64), indexing="ij"), -1).reshape(-1, 3)
    at_limit = np.concatenate([np.zeros((full.shape[0], 1), dtype=np.int64), full], 1).astype(np.int32)
    assert at_limit.shape[0] == 65536
    (nbr_a, pairs_a, num_a), (nbr_b, pairs_b, num_b) = _both(L, _ext, at_limit, 1, [16, 64, 64], [3] * 3, [1, 1, 1], cuda)
    assert np.array_equal(num_a, num_b) and np.array_equal(nbr_a, nbr_b) and np.array_equal(pairs_a, pairs_b)
    assert num_a[13] == 65536
    # a request beyond the built-in capacity is refused with a clear message, nothing is launched
    I3 = ctypes.c_int * 3
    rc = L.ssc_rulebook_subm_static(None, 70000, 1, I3(64, 64, 64), I3(3, 3, 3), I3(1, 1, 1), None, None, None, None,
                                    None)
    assert rc == 1 and b"65536" in L.ssc_last_error()
