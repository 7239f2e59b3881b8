"""Shared helpers of the GPU parity tests (the CUDA path is reached through ss_conv._ext,
i.e. ctypes calls into the C-ABI library)."""
import numpy as np
import torch

import ssconv_oracle as O


def dev(a, device, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(device)


def gpu_rulebook(ind, batch, shape, k, s, p, d, subm, device, transpose=False):
    from ss_conv.sp_ops.ops import get_indice_pairs
    outids, pairs, num = get_indice_pairs(dev(ind, device), batch, list(shape), k, s, p, d, 0, subm, transpose)
    return outids, pairs, num


def assert_rulebook_equal(gpu, ref):
    """Bit-exact after order normalisation (ascending outputs, pairs sorted by input row)."""
    g_out, g_pairs, g_num = (t.cpu().numpy() for t in gpu)
    r_out, r_pairs, r_num = ref
    assert g_pairs.shape == r_pairs.shape
    assert np.array_equal(g_num, r_num)
    cg = O.canonical_rulebook(g_out, g_pairs, g_num)
    cr = O.canonical_rulebook(r_out, r_pairs, r_num)
    assert np.array_equal(cg[0], cr[0])
    for a, b in zip(cg[1], cr[1]):
        assert np.array_equal(a, b)
    # padding beyond the count is -1 as in the reference layout
    for kappa in range(g_pairs.shape[0]):
        assert (g_pairs[kappa, :, g_num[kappa]:] == -1).all()
    # the GPU path numbers outputs by ascending flat index
    assert np.array_equal(g_out, cg[0])


def random_voxels(rng, batch, V, n_per_sample):
    rows = []
    for b in range(batch):
        flat = rng.choice(V ** 3, n_per_sample, replace=False)
        rows.append(np.stack([np.full(n_per_sample, b), flat // (V * V), (flat // V) % V, flat % V], 1))
    ind = np.concatenate(rows).astype(np.int32)
    return ind[O.renumber_rows(ind)]


def rel_err(a, ref):
    """max |a - ref| / max |ref| (per-tensor normalised error)."""
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(a, dtype=np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))
