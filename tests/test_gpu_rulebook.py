"""Rulebook kernels vs the CPU oracle: bit-exact after order normalisation."""
import numpy as np
import pytest
import torch

import ssconv_oracle as O
from gpu_helpers import assert_rulebook_equal, gpu_rulebook, random_voxels, dev

pytestmark = pytest.mark.gpu

CASES = [(3, 1, 1, 1, False), (3, 2, 1, 1, False), (2, 2, 0, 1, False), (3, 1, 0, 2, False), (3, 1, 1, 1, True),
         (5, 1, 2, 1, True), (3, 3, 2, 1, False), (3, 1, 1, 2, True), (5, 2, 2, 1, False), (1, 1, 0, 1, False)]


@pytest.mark.parametrize("table", ["dense", "hash"])
@pytest.mark.parametrize("k,s,p,d,subm", CASES)
def test_rulebook_matches_oracle(cuda, k, s, p, d, subm, table, monkeypatch):
    """Both ways of finding an input row: the dense row map over the input grid and the hash table."""
    from ss_conv import _ext
    monkeypatch.setenv("SSC_RULEBOOK_TABLE", table)
    _ext._scratch_cache.clear()            # scratch sizes depend on the table kind
    rng = np.random.RandomState(k * 100 + s * 10 + p + d)
    ind = random_voxels(rng, 3, 14, 300)
    try:
        got = gpu_rulebook(ind, 3, [14] * 3, k, s, p, d, subm, cuda)
    finally:
        _ext._scratch_cache.clear()
    ref = O.get_indice_pairs(ind, 3, [14] * 3, k, s, p, d, subm)
    assert_rulebook_equal(got, ref)
    from ss_conv import _ext
    _ext.check_status(cuda)


def test_rulebook_golden_fixture(cuda, golden):
    ind = golden["rb_indices"]
    for ci, (k, s, p, d, subm) in enumerate(golden["rb_cases"]):
        got = gpu_rulebook(ind, 2, [12] * 3, int(k), int(s), int(p), int(d), bool(subm), cuda)
        ref = (golden["rb%d_outids" % ci], golden["rb%d_pairs" % ci], golden["rb%d_num" % ci])
        assert_rulebook_equal(got, ref)


def test_rulebook_unsorted_input_and_anisotropic(cuda):
    rng = np.random.RandomState(5)
    ind = random_voxels(rng, 2, 10, 200)
    ind = ind[rng.permutation(ind.shape[0])]
    ind[:, 3] = ind[:, 3] % 7                      # z extent 7
    ind = np.unique(ind, axis=0)
    ind = ind[rng.permutation(ind.shape[0])].astype(np.int32)
    shape = [10, 10, 7]
    for subm in (False, True):
        got = gpu_rulebook(ind, 2, shape, [3, 2, 3], [1, 1, 1] if subm else [2, 1, 1], [1, 0, 1], 1, subm, cuda)
        ref = O.get_indice_pairs(ind, 2, shape, [3, 2, 3], [1, 1, 1] if subm else [2, 1, 1], [1, 0, 1], 1, subm)
        if subm:
            g_out, g_pairs, g_num = (t.cpu().numpy() for t in got)
            assert np.array_equal(g_out, ind) and np.array_equal(g_num, ref[2])
            for kappa in range(g_pairs.shape[0]):
                c = g_num[kappa]
                a = g_pairs[kappa, :, :c]
                b = ref[1][kappa, :, :c]
                assert np.array_equal(a[:, np.argsort(a[0])], b[:, np.argsort(b[0])])
        else:
            assert_rulebook_equal(got, ref)


def test_rulebook_empty_and_single(cuda):
    empty = np.zeros((0, 4), np.int32)
    out, pairs, num = gpu_rulebook(empty, 1, [8] * 3, 3, 1, 1, 1, False, cuda)
    assert out.shape == (0, 4) and pairs.shape == (27, 2, 0) and int(num.sum()) == 0
    out, pairs, num = gpu_rulebook(empty, 1, [8] * 3, 3, 1, 1, 1, True, cuda)
    assert out.shape == (0, 4) and int(num.sum()) == 0
    one = np.array([[0, 0, 0, 0]], np.int32)
    got = gpu_rulebook(one, 1, [4] * 3, 3, 1, 1, 1, False, cuda)
    assert_rulebook_equal(got, O.get_indice_pairs(one, 1, [4] * 3, 3, 1, 1, 1, False))
    full = np.stack(np.meshgrid(np.arange(1), np.arange(5), np.arange(5), np.arange(5), indexing="ij"), -1).reshape(-1, 4).astype(np.int32)
    got = gpu_rulebook(full, 1, [5] * 3, 3, 1, 1, 1, True, cuda)    # dense grid: maximum pair count
    assert_rulebook_equal(got, O.get_indice_pairs(full, 1, [5] * 3, 3, 1, 1, 1, True))


def test_rulebook_rejects_bad_input(cuda):
    from ss_conv import _ext
    bad = np.array([[0, 1, 2, 9]], np.int32)       # z outside an 8^3 grid
    gpu_rulebook(bad, 1, [8] * 3, 3, 1, 1, 1, True, cuda)
    with pytest.raises(RuntimeError):
        _ext.check_status(cuda)
    _ext.check_status(cuda)                        # the status word was cleared
    with pytest.raises(ValueError):                # kernel volume 343 > 256
        gpu_rulebook(np.zeros((1, 4), np.int32), 1, [8] * 3, 7, 1, 3, 1, True, cuda)
    with pytest.raises(ValueError):                # flat index does not fit int32
        gpu_rulebook(np.zeros((1, 4), np.int32), 64, [512] * 3, 3, 1, 1, 1, True, cuda)


def test_pairs_to_neighbour_table_and_inverse(cuda):
    """A reference-format rulebook given without the cached table, and the inverse-conv view."""
    from ss_conv import _ext
    rng = np.random.RandomState(11)
    ind = random_voxels(rng, 2, 10, 150)
    outids, pairs, num = O.get_indice_pairs(ind, 2, [10] * 3, 3, 2, 1, 1, False)
    n_out = outids.shape[0]
    nbr = _ext.neighbour_table(dev(pairs, cuda), dev(num, cuda), n_out).cpu().numpy()
    expect = np.full((27, n_out), -1, np.int32)
    for kappa in range(27):
        c = num[kappa]
        expect[kappa, pairs[kappa, 1, :c]] = pairs[kappa, 0, :c]
    assert np.array_equal(nbr, expect)
    inv = _ext.neighbour_table(dev(pairs, cuda), dev(num, cuda), ind.shape[0], inverse=True).cpu().numpy()
    expect = np.full((27, ind.shape[0]), -1, np.int32)
    for kappa in range(27):
        c = num[kappa]
        expect[kappa, pairs[kappa, 0, :c]] = pairs[kappa, 1, :c]
    assert np.array_equal(inv, expect)


def test_rulebook_full_size_properties(cuda):
    """Benchmark-size case (batch 32, 64^3, stride 2): properties that need no CPU oracle run."""
    from ss_conv.utils import synthetic as S
    ind = S.surface_voxels(range(32), 64, 16384, base_seed=1000)
    out, pairs, num = gpu_rulebook(ind, 32, [64] * 3, 3, 2, 1, 1, False, cuda)
    out, pairs, num = out.cpu().numpy(), pairs.cpu().numpy(), num.cpu().numpy()
    flat = ((out[:, 0].astype(np.int64) * 32 + out[:, 1]) * 32 + out[:, 2]) * 32 + out[:, 3]
    assert (np.diff(flat) > 0).all()                       # sorted, unique outputs
    total = 0
    for kappa in range(27):
        c = num[kappa]
        i, o = pairs[kappa, 0, :c], pairs[kappa, 1, :c]
        kk = np.array([kappa // 9, (kappa // 3) % 3, kappa % 3])
        assert np.array_equal(out[o, 1:] * 2 - 1 + kk, ind[i, 1:])      # geometry of every pair
        assert np.array_equal(out[o, 0], ind[i, 0])
        assert np.unique(i).size == c and np.unique(o).size == c
        total += c
    # every (input, offset) with a valid output appears: count from the closed form
    odd = (ind[:, 1:] % 2 == 1)
    per_dim = np.where(odd, 2, 1)
    # an odd coordinate reaches 2 outputs unless the upper one falls off the grid (coordinate 63 -> 32)
    per_dim = per_dim - ((ind[:, 1:] == 63) & odd)
    assert total == int(per_dim.prod(1).sum())
    assert np.unique(np.concatenate([pairs[k, 1, :num[k]] for k in range(27)])).size == out.shape[0]


def test_transposed_rulebook(cuda, golden):
    """Transposed convolution geometry vs the reference's own output and vs the oracle."""
    ind = golden["rbt_indices"]
    for ci, (k, s, p, op) in enumerate(golden["rbt_cases"]):
        from ss_conv.sp_ops.ops import get_indice_pairs
        got = get_indice_pairs(dev(ind, cuda), 2, [8] * 3, int(k), int(s), int(p), 1, int(op), False, True)
        ref = (golden["rbt%d_outids" % ci], golden["rbt%d_pairs" % ci], golden["rbt%d_num" % ci])
        assert_rulebook_equal(got, ref)
    rng = np.random.RandomState(9)
    big = random_voxels(rng, 2, 12, 300)
    got = gpu_rulebook(big, 2, [12] * 3, 3, 2, 1, 1, False, cuda, transpose=True)
    assert_rulebook_equal(got, O.get_indice_pairs(big, 2, [12] * 3, 3, 2, 1, 1, False, True, 0))


def test_lazy_pairs_materialise_to_the_same_lists(cuda):
    """Layers build rulebooks without pair lists; the handle must turn into exactly the lists
    the eager entry point produces."""
    from ss_conv.sp_ops.ops import get_indice_pairs
    rng = np.random.RandomState(17)
    ind = random_voxels(rng, 2, 12, 280)
    for subm, s in ((False, 2), (True, 1)):
        eager = get_indice_pairs(dev(ind, cuda), 2, [12] * 3, 3, s, 1, 1, 0, subm)
        lazy = get_indice_pairs(dev(ind, cuda), 2, [12] * 3, 3, s, 1, 1, 0, subm, lazy=True)
        assert lazy[1].shape == eager[1].shape and torch.equal(lazy[0], eager[0]) and torch.equal(lazy[2], eager[2])
        assert torch.equal(lazy[1].materialize(), eager[1])
        assert torch.equal(lazy[1][3], eager[1][3])          # tensor behaviour on demand


@pytest.mark.parametrize("order", ["by_sample", "shuffled"])
def test_rulebook_on_a_coarse_grid_with_many_samples(cuda, order):
    """Coarse output grids mark their cells through a per-block image of bitmap words when a block's
    rows belong to few samples (rows ordered by sample) and directly when they do not (shuffled rows
    of 40 samples span more words than the image holds): same rulebook either way."""
    rng = np.random.RandomState(77)
    ind = random_voxels(rng, 40, 16, 260)
    if order == "shuffled":
        ind = ind[rng.permutation(ind.shape[0])]
    ind = np.ascontiguousarray(ind.astype(np.int32))
    for k, s, p in ((3, 1, 1), (3, 2, 1), (2, 2, 0)):
        got = gpu_rulebook(ind, 40, [16] * 3, k, s, p, 1, False, cuda)
        ref = O.get_indice_pairs(ind, 40, [16] * 3, k, s, p, 1, False)
        assert_rulebook_equal(got, ref)
    from ss_conv import _ext
    _ext.check_status(cuda)
