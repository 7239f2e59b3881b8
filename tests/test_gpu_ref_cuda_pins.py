"""Three-way pins for the helper ops that have no CPU implementation in the reference: the
reference's OWN CUDA kernels (its extension compiled from SS_Conv_lib/src into oracle/_ref, called
here on CUDA tensors) vs the numpy restatement in oracle/ssconv_oracle.py vs this library's C ABI.

One function per test so that a failure names itself.  Inputs are small (a few thousand rows).
Reference sources pinned: pool/indice_avgpool_cuda_functor.cu:21-53, pool/indiceSummaryRF.cu:21-36,
pool/global_avgpool_cuda_kernel.cu:16-60, pool/global_maxpool_cuda_kernel.cu:16-60,
voxelize/voxel2point_cuda_kernel.cu:16-37, voxelize/voxelize_cuda_kernel.h:18-60,
voxelize/interpolate_cuda_kernel.cu:8-140, conv/indice_cuda_functor.cu:23-345,
conv/indice_conv.h:247-426.
"""
import numpy as np
import pytest
import torch

import ssconv_oracle as O
from gpu_helpers import dev, gpu_rulebook, random_voxels, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(cuda):
    from ref_loader import load_ref_ext
    m = load_ref_ext()
    if m is None:
        pytest.skip("the reference extension (oracle/_ref) has not been built: python oracle/build_ref.py")
    return m


def _pool_case(cuda, c, seed, k=3, s=2, p=1):
    rng = np.random.RandomState(seed)
    ind = random_voxels(rng, 3, 12, 500)
    feats = rng.randn(ind.shape[0], c).astype(np.float32)
    outids, pairs, num = gpu_rulebook(ind, 3, [12] * 3, k, s, p, 1, False, cuda)
    return ind, feats, outids, pairs.contiguous(), num.contiguous()


@pytest.mark.parametrize("c", [64, 30])
def test_ref_cuda_summary_rf(cuda, ref, c):
    from ss_conv import _ext
    ind, feats, outids, pairs, num = _pool_case(cuda, c, 11)
    n_out = outids.shape[0]
    r = ref.indiceSummaryRF(pairs, num, n_out).cpu().numpy()
    o = O.summary_rf(pairs.cpu().numpy(), num.cpu().numpy(), n_out)
    g = _ext.indiceSummaryRF(pairs, num, n_out).cpu().numpy()
    assert np.array_equal(r, o) and np.array_equal(g, r)


@pytest.mark.parametrize("c", [64, 30, 3])
@pytest.mark.parametrize("use_gs", [True, False])
def test_ref_cuda_avgpool_forward(cuda, ref, c, use_gs):
    from ss_conv import _ext
    ind, feats, outids, pairs, num = _pool_case(cuda, c, 12 + c)
    n_out = outids.shape[0]
    pn, nn = pairs.cpu().numpy(), num.cpu().numpy()
    if use_gs:   # the Python default: divisor = kernel volume (sp_ops/functional.py:171-176)
        rf = torch.full((n_out,), pairs.shape[0], dtype=torch.int32, device=cuda)
    else:
        rf = ref.indiceSummaryRF(pairs, num, n_out)
    f = dev(feats, cuda)
    r = ref.indice_avgpool_fp32(f, pairs, num, n_out, rf).cpu().numpy()
    o = O.indice_avgpool(feats, pn, nn, n_out, rf.cpu().numpy())
    g = _ext.indice_avgpool_fp32(f, pairs, num, n_out, rf).cpu().numpy()
    assert np.array_equal(r, o), "oracle restatement differs from the reference CUDA kernel"
    assert np.array_equal(g, r), "library differs from the reference CUDA kernel"


@pytest.mark.parametrize("c", [64, 30])
def test_ref_cuda_avgpool_backward(cuda, ref, c):
    from ss_conv import _ext
    ind, feats, outids, pairs, num = _pool_case(cuda, c, 40 + c)
    n_out = outids.shape[0]
    rf = ref.indiceSummaryRF(pairs, num, n_out)
    f = dev(feats, cuda)
    y = ref.indice_avgpool_fp32(f, pairs, num, n_out, rf)
    gy = torch.randn_like(y)
    r = ref.indice_avgpool_backward_fp32(f, y, gy, pairs, num, rf).cpu().numpy()
    g = _ext.indice_avgpool_backward_fp32(f, y, gy, pairs, num, rf).cpu().numpy()
    o = O.indice_avgpool_backward(feats, gy.cpu().numpy(), pairs.cpu().numpy(), num.cpu().numpy(), rf.cpu().numpy())
    assert np.array_equal(r, o), "oracle restatement differs from the reference CUDA kernel"
    assert np.array_equal(g, r), "library differs from the reference CUDA kernel"


def _segments(rng, counts, c):
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    feats = rng.randn(int(off[-1]), c).astype(np.float32)
    return feats, off


@pytest.mark.parametrize("c", [240, 70, 5])
def test_ref_cuda_global_avgpool(cuda, ref, c):
    from ss_conv import _ext
    rng = np.random.RandomState(c)
    feats, off = _segments(rng, [37, 1, 200, 64, 9, 513], c)
    B = len(off) - 1
    f, o_ = dev(feats, cuda), dev(off, cuda)
    r_out = torch.zeros(B, c, device=cuda)
    r_idx = torch.zeros(B, c, dtype=torch.int32, device=cuda)
    ref.global_avgpool_fp(f, o_, r_out, r_idx, B, c)
    torch.cuda.synchronize()
    g_out = torch.zeros(B, c, device=cuda)
    _ext.global_avgpool_fp(f, o_, g_out, torch.zeros(B, c, dtype=torch.int32, device=cuda), B, c)
    r = r_out.cpu().numpy()
    assert np.array_equal(r, O.global_avgpool(feats, off)), "oracle (sequential fp32 row sum) differs from the reference kernel"
    # the library sums the rows of a sample pairwise, not one after the other: tolerance, not bits
    assert np.abs(g_out.cpu().numpy() - r).max() <= 2e-6 * np.abs(feats).max() * np.sqrt(513)
    # backward: d_feats[row] = d_out[sample] / len
    d_out = torch.randn(B, c, device=cuda)
    r_d = torch.zeros(feats.shape[0], c, device=cuda)
    g_d = torch.zeros(feats.shape[0], c, device=cuda)
    ref.global_avgpool_bp(r_d, o_, r_idx, d_out, B, c)
    torch.cuda.synchronize()
    _ext.global_avgpool_bp(g_d, o_, r_idx, d_out, B, c)
    assert np.array_equal(g_d.cpu().numpy(), r_d.cpu().numpy())
    assert np.array_equal(r_d.cpu().numpy(), O.global_avgpool_backward(d_out.cpu().numpy(), off, feats.shape[0]))


@pytest.mark.parametrize("c", [240, 70, 5])
def test_ref_cuda_global_maxpool(cuda, ref, c):
    from ss_conv import _ext
    rng = np.random.RandomState(100 + c)
    feats, off = _segments(rng, [37, 1, 200, 64, 9, 513], c)
    feats[40:60] = feats[38:39]          # ties inside a sample: the first row must win
    B = len(off) - 1
    f, o_ = dev(feats, cuda), dev(off, cuda)
    r_out, g_out = torch.zeros(B, c, device=cuda), torch.zeros(B, c, device=cuda)
    r_idx = torch.zeros(B, c, dtype=torch.int32, device=cuda)
    g_idx = torch.zeros(B, c, dtype=torch.int32, device=cuda)
    ref.global_maxpool_fp(f, o_, r_out, r_idx, B, c)
    torch.cuda.synchronize()
    _ext.global_maxpool_fp(f, o_, g_out, g_idx, B, c)
    o_out, o_idx = O.global_maxpool(feats, off)
    assert np.array_equal(r_out.cpu().numpy(), o_out) and np.array_equal(r_idx.cpu().numpy(), o_idx)
    assert np.array_equal(g_out.cpu().numpy(), r_out.cpu().numpy())
    assert np.array_equal(g_idx.cpu().numpy(), r_idx.cpu().numpy())
    d_out = torch.randn(B, c, device=cuda)
    r_d = torch.zeros(feats.shape[0], c, device=cuda)
    g_d = torch.zeros(feats.shape[0], c, device=cuda)
    ref.global_maxpool_bp(r_d, o_, r_idx, d_out, B, c)
    torch.cuda.synchronize()
    _ext.global_maxpool_bp(g_d, o_, g_idx, d_out, B, c)
    assert np.array_equal(g_d.cpu().numpy(), r_d.cpu().numpy())
    assert np.array_equal(r_d.cpu().numpy(), O.global_maxpool_backward(d_out.cpu().numpy(), o_idx, feats.shape[0]))


def _sorted_lists(maps, mode):
    """Rows [count, ids...] with the id list sorted (modes 3/4 append in atomic order in the
    reference); the unused tail of a row is left as the reference initialised it."""
    maps = maps.copy()
    if mode in (3, 4):
        for v in range(maps.shape[0]):
            c = maps[v, 0]
            maps[v, 1:1 + c] = np.sort(maps[v, 1:1 + c])
    return maps


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
def test_ref_cuda_voxel2point_map(cuda, ref, mode):
    from ss_conv import _ext
    rng = np.random.RandomState(mode)
    n, m = 3000, 400
    inverse = rng.randint(0, m, n).astype(np.int32)
    inverse[:m] = np.arange(m)
    max_active = 1 if mode in (1, 2) else int(np.bincount(inverse, minlength=m).max())
    init = {1: n, 2: -1, 3: 0, 4: 0}[mode]          # sp_ops/functional.py:344-351
    inv = dev(inverse, cuda)
    ids = torch.arange(n, dtype=torch.int32, device=cuda)
    r_maps = torch.full((m, max_active + 1), init, dtype=torch.int32, device=cuda)
    g_maps = r_maps.clone()
    ref.voxel2point_map(inv, ids, r_maps, n, max_active, mode)
    torch.cuda.synchronize()
    _ext.voxel2point_map(inv, ids, g_maps, n, max_active, mode)
    r = _sorted_lists(r_maps.cpu().numpy(), mode)
    assert np.array_equal(r, O.voxel2point_map(inverse, m, max_active, mode))
    assert np.array_equal(g_maps.cpu().numpy(), r)     # the library writes ascending ids: already sorted


@pytest.mark.parametrize("mode", [3, 4, 1])
@pytest.mark.parametrize("c", [3, 19])
def test_ref_cuda_voxelize_fp_and_bp(cuda, ref, mode, c):
    from ss_conv import _ext
    rng = np.random.RandomState(10 * mode + c)
    n, m = 3000, 400
    inverse = rng.randint(0, m, n).astype(np.int32)
    inverse[:m] = np.arange(m)
    max_active = 1 if mode in (1, 2) else int(np.bincount(inverse, minlength=m).max())
    maps_np = O.voxel2point_map(inverse, m, max_active, mode)
    maps = dev(maps_np, cuda)
    feats = rng.rand(n, c).astype(np.float32)
    f = dev(feats, cuda)
    r_out, g_out = torch.zeros(m, c, device=cuda), torch.zeros(m, c, device=cuda)
    ref.voxelize_fp(f, r_out, maps, mode, m, max_active, c)
    torch.cuda.synchronize()
    _ext.voxelize_fp(f, g_out, maps, mode, m, max_active, c)
    assert np.array_equal(r_out.cpu().numpy(), O.voxelize_fp(feats, maps_np, mode))
    assert np.array_equal(g_out.cpu().numpy(), r_out.cpu().numpy())
    d_out = torch.randn(m, c, device=cuda)
    r_d, g_d = torch.zeros(n, c, device=cuda), torch.zeros(n, c, device=cuda)
    ref.voxelize_bp(d_out, r_d, maps, mode, m, max_active, c)
    torch.cuda.synchronize()
    _ext.voxelize_bp(d_out, g_d, maps, mode, m, max_active, c)
    assert np.array_equal(g_d.cpu().numpy(), r_d.cpu().numpy())
    assert np.array_equal(r_d.cpu().numpy(), O.voxelize_bp(d_out.cpu().numpy(), maps_np, mode, n))


def _nn_case(rng, n, m, batch, V=16):
    """Queries = random points, known = centres of random voxels of a V^3 grid (many equal
    distances: a regular grid is where tie order and last-bit rounding show)."""
    kb = np.sort(rng.randint(0, batch, m))
    cells = rng.randint(0, V, (m, 3))
    known = np.concatenate([kb[:, None], (cells + 0.5) / V - 0.5], 1).astype(np.float32)
    ub = np.sort(rng.randint(0, batch, n))
    unknown = np.concatenate([ub[:, None], rng.uniform(-0.5, 0.5, (n, 3))], 1).astype(np.float32)
    unknown[: n // 4, 1:] = (np.round(unknown[: n // 4, 1:] * V) / V).astype(np.float32)   # on cell corners: exact ties
    return unknown, known


def test_ref_cuda_three_nn(cuda, ref):
    from ss_conv import _ext
    rng = np.random.RandomState(5)
    unknown, known = _nn_case(rng, 4000, 2500, 4)
    u, k = dev(unknown, cuda), dev(known, cuda)
    n, m = unknown.shape[0], known.shape[0]
    r_d, g_d = torch.zeros(n, 3, device=cuda), torch.zeros(n, 3, device=cuda)
    r_i = torch.zeros(n, 3, dtype=torch.int32, device=cuda)
    g_i = torch.zeros(n, 3, dtype=torch.int32, device=cuda)
    ref.three_nn(n, m, u, k, r_d, r_i)
    torch.cuda.synchronize()
    _ext.three_nn(n, m, u, k, g_d, g_i)
    o_d, o_i = O.three_nn(unknown, known)
    assert np.array_equal(r_i.cpu().numpy(), o_i), "oracle neighbours differ from the reference kernel"
    assert np.array_equal(r_d.cpu().numpy(), o_d), "oracle distances differ from the reference kernel (bitwise)"
    assert np.array_equal(g_i.cpu().numpy(), r_i.cpu().numpy()), "library neighbours differ from the reference kernel"
    assert np.array_equal(g_d.cpu().numpy(), r_d.cpu().numpy()), "library distances differ from the reference kernel (bitwise)"


@pytest.mark.parametrize("c", [19, 64])
def test_ref_cuda_three_interpolate(cuda, ref, c):
    from ss_conv import _ext
    rng = np.random.RandomState(c)
    n, m = 3000, 700
    pts = rng.randn(m, c).astype(np.float32)
    idx = rng.randint(0, m, (n, 3)).astype(np.int32)
    w = rng.rand(n, 3).astype(np.float32)
    w /= w.sum(1, keepdims=True)
    p, i_, w_ = dev(pts, cuda), dev(idx, cuda), dev(w, cuda)
    r_out, g_out = torch.zeros(n, c, device=cuda), torch.zeros(n, c, device=cuda)
    ref.three_interpolate_fp(c, m, n, p, i_, w_, r_out)
    torch.cuda.synchronize()
    _ext.three_interpolate_fp(c, m, n, p, i_, w_, g_out)
    assert np.array_equal(r_out.cpu().numpy(), O.three_interpolate(pts, idx, w)), "oracle differs from the reference kernel (bitwise)"
    assert np.array_equal(g_out.cpu().numpy(), r_out.cpu().numpy()), "library differs from the reference kernel (bitwise)"
    # backward: float atomics in both the reference and the library -> order-dependent rounding
    gy = torch.randn(n, c, device=cuda)
    r_g, g_g = torch.zeros(m, c, device=cuda), torch.zeros(m, c, device=cuda)
    ref.three_interpolate_bp(c, n, m, gy, i_, w_, r_g)
    torch.cuda.synchronize()
    _ext.three_interpolate_bp(c, n, m, gy, i_, w_, g_g)
    o_g = O.three_interpolate_bp(gy.cpu().numpy(), idx, w, m)
    assert rel_err(r_g.cpu().numpy(), o_g) <= 2e-6
    assert rel_err(g_g.cpu().numpy(), o_g) <= 2e-6


# ---------------------------------------------------------------- rulebook / conv / max pool on CUDA
def test_ref_cuda_rulebook_conv_maxpool(cuda, ref):
    """The reference's CUDA rulebook, gather-GEMM-scatter and max pool (the SIMT + cuBLAS path the
    library replaces) against the library on the same CUDA tensors."""
    from ss_conv import _ext
    rng = np.random.RandomState(21)
    B, V, k, s, p = 3, 16, 3, 2, 1
    ind = random_voxels(rng, B, V, 900)
    ci, co = 32, 38
    feats = rng.randn(ind.shape[0], ci).astype(np.float32)
    W = (rng.randn(k, k, k, ci, co) / np.sqrt(ci * k ** 3)).astype(np.float32)
    osz = O.conv_output_size([V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3)
    ti = dev(ind, cuda)
    r_out, r_pairs, r_num = ref.get_indice_pairs_3d(ti, B, osz, [V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3, [0] * 3, 0, 0)
    g_out, g_pairs, g_num = _ext.get_indice_pairs_3d(ti, B, osz, [V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3, [0] * 3, 0, 0)
    cr = O.canonical_rulebook(r_out.cpu().numpy(), r_pairs.cpu().numpy(), r_num.cpu().numpy())
    cg = O.canonical_rulebook(g_out.cpu().numpy(), g_pairs.cpu().numpy(), g_num.cpu().numpy())
    assert np.array_equal(r_num.cpu().numpy(), g_num.cpu().numpy())
    assert np.array_equal(cr[0], cg[0])
    for a, b in zip(cr[1], cg[1]):
        assert np.array_equal(a, b)
    assert np.array_equal(r_out.cpu().numpy(), g_out.cpu().numpy())     # both number outputs by ascending flat index
    f, w = dev(feats, cuda), dev(W, cuda)
    n_out = r_out.shape[0]
    y_ref = ref.indice_conv_fp32(f, w, r_pairs, r_num, n_out, 0, 0).cpu().numpy()
    prev = _ext.get_precision()
    try:
        _ext.set_precision("fp32")
        y32 = _ext.indice_conv_fp32(f, w, g_pairs, g_num, n_out, 0, 0).cpu().numpy()
        _ext.set_precision("tf32")
        ytc = _ext.indice_conv_fp32(f, w, g_pairs, g_num, n_out, 0, 0).cpu().numpy()
    finally:
        _ext.set_precision(prev)
    y64 = O.indice_conv(feats.astype(np.float64), W.astype(np.float64), g_pairs.cpu().numpy(), g_num.cpu().numpy(), n_out)
    assert rel_err(y_ref, y64) <= 2e-5      # the reference's cuBLAS GEMM may itself use TF32-free fp32
    assert rel_err(y32, y_ref) <= 2e-5
    assert rel_err(ytc, y_ref) <= 1e-3      # TF32 operands: the north-star tolerance
    # max pool k2 s2 on the conv output, reference CUDA vs library, bit-exact
    psz = O.conv_output_size(osz, [2] * 3, [2] * 3, [0] * 3, [1] * 3)
    yr = torch.from_numpy(y_ref).to(cuda)
    p_out, p_pairs, p_num = ref.get_indice_pairs_3d(r_out.contiguous(), B, psz, osz, [2] * 3, [2] * 3, [0] * 3, [1] * 3, [0] * 3, 0, 0)
    q_out, q_pairs, q_num = _ext.get_indice_pairs_3d(g_out.contiguous(), B, psz, osz, [2] * 3, [2] * 3, [0] * 3, [1] * 3, [0] * 3, 0, 0)
    m_ref = ref.indice_maxpool_fp32(yr, p_pairs, p_num, p_out.shape[0]).cpu().numpy()
    m_lib = _ext.indice_maxpool_fp32(yr, q_pairs, q_num, q_out.shape[0]).cpu().numpy()
    assert np.array_equal(p_out.cpu().numpy(), q_out.cpu().numpy())
    assert np.array_equal(m_ref, m_lib)
