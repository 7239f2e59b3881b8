"""Random geometries, orders and channel counts: rulebook bit-exact against the CPU oracle, the
convolution in every operand precision against a float64 evaluation of the same table, the pools
and the voxelizer bit-exact against the oracle.

Tolerances (max |diff| / max |ref|) are wider than in the layer-sized tests because many cases are a
handful of rows and terms, where one operand's rounding is not averaged out: exact fp32 1e-4, TF32 and
fp16 operands 4e-3, bf16 operands 4e-2.  An indexing fault shows as an error of order one."""
import numpy as np
import pytest
import torch

import ssconv_oracle as O
from gpu_helpers import assert_rulebook_equal, gpu_rulebook

pytestmark = pytest.mark.gpu
TOL = (("fp32", 1e-4), ("tf32", 4e-3), ("fp16", 4e-3), ("bf16", 4e-2))


def _random_case(rng):
    batch = int(rng.randint(1, 6))
    V = [int(rng.randint(3, 20)) for _ in range(3)]
    k = [int(rng.randint(1, 4)) for _ in range(3)]
    s = [int(rng.randint(1, 3)) for _ in range(3)]
    d = [1 if s[i] > 1 else int(rng.randint(1, 3)) for i in range(3)]
    p = [int(rng.randint(0, k[i])) for i in range(3)]
    subm = bool(rng.rand() < 0.3) and all(x % 2 == 1 for x in k)
    if subm:
        s, p = [1, 1, 1], [(k[i] // 2) * d[i] for i in range(3)]
    cells = V[0] * V[1] * V[2]
    per = min(int(rng.randint(1, max(2, min(cells, 600)))), cells)
    rows = []
    for b in range(batch):
        flat = rng.choice(cells, per, replace=False)
        rows.append(np.stack([np.full(per, b), flat // (V[1] * V[2]), (flat // V[2]) % V[1], flat % V[2]], 1))
    ind = np.concatenate(rows).astype(np.int32)
    ind = ind[rng.permutation(ind.shape[0])] if rng.rand() < 0.5 else ind[O.renumber_rows(ind)]
    out_shape = [(V[i] + 2 * p[i] - d[i] * (k[i] - 1) - 1) // s[i] + 1 for i in range(3)]
    return (batch, V, k, s, p, d, subm, np.ascontiguousarray(ind)) if min(out_shape) >= 1 else None


@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_random_geometries_against_the_oracle(cuda, seed):
    from ss_conv import _ext
    rng = np.random.RandomState(seed)
    done = 0
    while done < 120:
        case = _random_case(rng)
        if case is None:
            continue
        batch, V, k, s, p, d, subm, ind = case
        got = gpu_rulebook(ind, batch, V, k, s, p, d, subm, cuda)
        ref = O.get_indice_pairs(ind, batch, V, k, s, p, d, subm)
        what = (k, s, p, d, subm, V, ind.shape[0])
        if subm:
            assert np.array_equal(got[2].cpu().numpy(), ref[2]), what
        else:
            assert_rulebook_equal(got, ref)
        outids, pairs, num = got
        n_out = outids.shape[0]
        done += 1
        if n_out == 0:
            continue
        c_in = int(rng.choice([1, 3, 4, 7, 8, 16, 20, 32, 33, 64, 100]))
        c_out = int(rng.choice([1, 5, 16, 38, 76, 130, 260]))
        K = k[0] * k[1] * k[2]
        f = torch.randn(ind.shape[0], c_in, device=cuda)
        W = torch.randn(K, c_in, c_out, device=cuda) / float(np.sqrt(c_in * K))
        nbr = _ext.neighbour_table(pairs, num, n_out)
        t, fd, Wd = nbr.cpu().numpy(), f.double().cpu().numpy(), W.double().cpu().numpy()
        want = np.zeros((n_out, c_out))
        for kap in range(K):
            m = t[kap] >= 0
            want[m] += fd[t[kap][m]] @ Wd[kap]
        scale = max(float(np.abs(want).max()), 1e-30)
        for prec, tol in TOL:
            y = _ext.conv_forward(f, W, nbr, n_out, prec).double().cpu().numpy()
            err = float(np.abs(y - want).max()) / scale
            assert err < tol, (prec, err, c_in, c_out) + what
        if not subm:     # the same rulebook drives the pools: bit-exact (same accumulation order)
            fn, pn, nn = f.cpu().numpy(), pairs.cpu().numpy(), num.cpu().numpy()
            assert np.array_equal(_ext.indice_maxpool_fp32(f, pairs, num, n_out).cpu().numpy(),
                                  O.indice_maxpool(fn, pn, nn, n_out)), ("maxpool", c_in) + what
            rf = _ext.indiceSummaryRF(pairs, num, n_out)
            assert np.array_equal(rf.cpu().numpy(), O.summary_rf(pn, nn, n_out)), ("summary", c_in) + what
            assert np.array_equal(_ext.indice_avgpool_fp32(f, pairs, num, n_out, rf).cpu().numpy(),
                                  O.indice_avgpool(fn, pn, nn, n_out, O.summary_rf(pn, nn, n_out))), ("avgpool", c_in) + what
    _ext.check_status(cuda)


@pytest.mark.parametrize("seed", [21, 22])
def test_random_point_clouds_through_the_voxelizer(cuda, seed):
    """Point2Voxel on random clouds (grid size, points per sample, feature count, mode, points outside
    the grid): voxels, features and ids as the oracle's."""
    from ss_conv import _ext
    from ss_conv.sp_ops.voxelize import Point2Voxel
    rng = np.random.RandomState(seed)
    for _ in range(40):
        B, V, mode = int(rng.randint(1, 6)), int(rng.choice([4, 8, 16, 32])), int(rng.randint(1, 5))
        per, C = int(rng.randint(1, 900)), int(rng.choice([1, 3, 4, 6, 9]))
        pts = rng.uniform(-0.55, 0.55, (B * per, 3)).astype(np.float32)      # ~25 % of the points fall outside
        pts[::per] = 0.01                                                    # every sample keeps a point (the oracle
                                                                             # does not restate the empty-sample branch)
        fts = rng.rand(B * per, C).astype(np.float32)
        ids = np.repeat(np.arange(B), per)
        p2v = Point2Voxel([V] * 3, [1.0 / V] * 3, mode)
        t = lambda a: torch.from_numpy(a).to(cuda)
        vp, sp, vids, flag = p2v(t(pts), t(fts), t(ids))
        rp, rfeat, rocc, rids, rinv = O.point2voxel(pts, fts, ids, [V] * 3, [1.0 / V] * 3, mode)
        what = (B, V, mode, per, C)
        assert np.array_equal(vp.cpu().numpy(), rp) and np.array_equal(vids.cpu().numpy(), rids), what
        assert np.array_equal(sp.indices.cpu().numpy(), rocc), what
        assert np.array_equal(sp.features.cpu().numpy(), rfeat), what
    _ext.check_status(cuda)


@pytest.mark.parametrize("seed", [31, 32])
def test_random_geometries_backward_against_float64(cuda, seed):
    """Both gradients of random convolutions.  The error of every entry is measured against the sum of
    the absolute values of its terms (so that a gradient that nearly cancels does not inflate it): exact
    fp32 2e-6, TF32 operands 1.5e-3 (two operands rounded to 11 bits each bound it by 2^-10)."""
    from ss_conv import _ext
    rng = np.random.RandomState(seed)
    done = 0
    while done < 100:
        case = _random_case(rng)
        if case is None:
            continue
        batch, V, k, s, p, d, subm, ind = case
        outids, pairs, num = gpu_rulebook(ind, batch, V, k, s, p, d, subm, cuda)
        n_out, n_in = outids.shape[0], ind.shape[0]
        done += 1
        if n_out == 0:
            continue
        c_in, c_out = int(rng.choice([1, 3, 4, 8, 16, 20, 32, 64])), int(rng.choice([1, 5, 16, 38, 76, 130]))
        K = k[0] * k[1] * k[2]
        f = torch.randn(n_in, c_in, device=cuda)
        W = torch.randn(K, c_in, c_out, device=cuda) / float(np.sqrt(c_in * K))
        g = torch.randn(n_out, c_out, device=cuda)
        nbr = _ext.neighbour_table(pairs, num, n_out)
        t, fd, Wd, gd = nbr.cpu().numpy(), f.double().cpu().numpy(), W.double().cpu().numpy(), g.double().cpu().numpy()
        din, dw = np.zeros((n_in, c_in)), np.zeros((K, c_in, c_out))
        din_abs, dw_abs = np.zeros((n_in, c_in)), np.zeros((K, c_in, c_out))
        for kap in range(K):
            m = np.nonzero(t[kap] >= 0)[0]
            if m.size == 0:
                continue
            src = t[kap][m]
            np.add.at(din, src, gd[m] @ Wd[kap].T)
            np.add.at(din_abs, src, np.abs(gd[m]) @ np.abs(Wd[kap]).T)
            dw[kap] = fd[src].T @ gd[m]
            dw_abs[kap] = np.abs(fd[src]).T @ np.abs(gd[m])
        for prec, tol in (("fp32", 2e-6), ("tf32", 1.5e-3)):
            a, b = _ext.conv_backward(f, W, g, nbr, precision=prec)
            e_in = float((np.abs(a.double().cpu().numpy() - din) / np.maximum(din_abs, 1e-30)).max())
            e_w = float((np.abs(b.double().cpu().numpy() - dw) / np.maximum(dw_abs, 1e-30)).max())
            assert e_in < tol and e_w < tol, (prec, e_in, e_w, k, s, p, d, subm, V, c_in, c_out, n_in, n_out)
    _ext.check_status(cuda)
