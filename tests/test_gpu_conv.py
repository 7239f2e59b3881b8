"""Gather-GEMM kernels vs the oracle.  Tolerances: exact-fp32 path 2e-5 (summation order
differs from the reference's GEMM), TF32 tensor-core path 1e-3, both as max|diff|/max|ref|
against the float64 evaluation of the same contraction."""
import numpy as np
import pytest
import torch

import ssconv_oracle as O
from gpu_helpers import dev, gpu_rulebook, random_voxels, rel_err

pytestmark = pytest.mark.gpu
# fp16 operands carry the same 11-bit significand as TF32
TOL = {"fp32": 2e-5, "tf32": 1e-3, "fp16": 1e-3, "bf16": 1e-2}    # max|err| / max|ref|; the bf16 / TF32 figures are the stated targets


def _run(cuda, ind, batch, V, k, s, p, subm, c_in, c_out, precision, seed=0):
    from ss_conv import _ext
    rng = np.random.RandomState(seed)
    feats = rng.randn(ind.shape[0], c_in).astype(np.float32)
    W = (rng.randn(k, k, k, c_in, c_out) / np.sqrt(c_in * k ** 3)).astype(np.float32)
    outids, pairs, num = gpu_rulebook(ind, batch, [V] * 3, k, s, p, 1, subm, cuda)
    _ext.set_precision(precision)
    try:
        y = _ext.indice_conv_fp32(dev(feats, cuda), dev(W, cuda), pairs, num, outids.shape[0], 0, int(subm))
        torch.cuda.synchronize()
        _ext.check_status(cuda)
    finally:
        _ext.set_precision("auto")
    ref = O.indice_conv_f64(feats, W, pairs.cpu().numpy(), num.cpu().numpy(), outids.shape[0])
    return y.cpu().numpy(), ref


@pytest.mark.parametrize("precision", ["fp32", "tf32"])
@pytest.mark.parametrize("c_in,c_out", [(32, 38), (64, 76), (3, 36), (30, 72), (16, 16), (130, 270)])
def test_conv_channel_shapes(cuda, precision, c_in, c_out):
    rng = np.random.RandomState(c_in + c_out)
    ind = random_voxels(rng, 2, 12, 330)           # > 2 row tiles, ragged last tile
    y, ref = _run(cuda, ind, 2, 12, 3, 1, 1, False, c_in, c_out, precision)
    assert rel_err(y, ref) <= TOL[precision]


@pytest.mark.parametrize("precision", ["fp32", "tf32"])
@pytest.mark.parametrize("k,s,p,subm", [(3, 2, 1, False), (3, 1, 1, True), (5, 1, 2, True), (2, 2, 0, False)])
def test_conv_geometries(cuda, precision, k, s, p, subm):
    rng = np.random.RandomState(k * 7 + s)
    ind = random_voxels(rng, 3, 14, 400)
    y, ref = _run(cuda, ind, 3, 14, k, s, p, subm, 32, 48, precision)
    assert rel_err(y, ref) <= TOL[precision]


def test_conv_fp32_matches_reference_oracle_tightly(cuda):
    rng = np.random.RandomState(1)
    ind = random_voxels(rng, 2, 10, 200)
    feats = rng.randn(ind.shape[0], 20).astype(np.float32)
    W = rng.randn(3, 3, 3, 20, 24).astype(np.float32)
    from ss_conv import _ext
    outids, pairs, num = gpu_rulebook(ind, 2, [10] * 3, 3, 1, 1, 1, True, cuda)
    _ext.set_precision("fp32")
    try:
        y = _ext.indice_conv_fp32(dev(feats, cuda), dev(W, cuda), pairs, num, ind.shape[0], 0, 1).cpu().numpy()
    finally:
        _ext.set_precision("auto")
    ref = O.indice_conv(feats, W, pairs.cpu().numpy(), num.cpu().numpy(), ind.shape[0], False, True)
    assert rel_err(y, ref) <= 2e-6


def test_inverse_conv(cuda):
    """Inverse convolution: the strided layer's rulebook with the pair roles exchanged."""
    from ss_conv import _ext
    rng = np.random.RandomState(2)
    ind = random_voxels(rng, 2, 12, 250)
    outids, pairs, num = gpu_rulebook(ind, 2, [12] * 3, 3, 2, 1, 1, False, cuda)
    n_out = outids.shape[0]
    feats = rng.randn(n_out, 16).astype(np.float32)
    W = rng.randn(3, 3, 3, 16, 24).astype(np.float32)
    for precision in ("fp32", "tf32"):
        _ext.set_precision(precision)
        try:
            y = _ext.indice_conv_fp32(dev(feats, cuda), dev(W, cuda), pairs, num, ind.shape[0], 1, 0).cpu().numpy()
        finally:
            _ext.set_precision("auto")
        ref = O.indice_conv_f64(feats, W, pairs.cpu().numpy(), num.cpu().numpy(), ind.shape[0], inverse=True)
        assert rel_err(y, ref) <= TOL[precision]


def test_inverse_conv_with_grouped_rows_gives_the_same_bits(cuda, monkeypatch):
    """A large inverse convolution runs through the row order of its table (rows grouped by parity
    class); the result is the one of the plain order, bit for bit."""
    from ss_conv import _ext
    rng = np.random.RandomState(3)
    ind = random_voxels(rng, 3, 32, 6000)
    outids, pairs, num = gpu_rulebook(ind, 3, [32] * 3, 3, 2, 1, 1, False, cuda)
    assert ind.shape[0] >= _ext.ROW_ORDER_MIN_ROWS
    feats = torch.randn(outids.shape[0], 32, device=cuda)
    W = torch.randn(3, 3, 3, 32, 24, device=cuda) / 20
    _ext.set_precision("tf32")
    try:
        l0 = _ext.kernel_launches()
        grouped = _ext.indice_conv_fp32(feats, W, pairs, num, ind.shape[0], 1, 0)
        l1 = _ext.kernel_launches()
        monkeypatch.setattr(_ext, "ROW_ORDER_MIN_ROWS", 1 << 30)
        plain = _ext.indice_conv_fp32(feats, W, pairs, num, ind.shape[0], 1, 0)
        l2 = _ext.kernel_launches()
        torch.cuda.synchronize()
        _ext.check_status(cuda)
    finally:
        _ext.set_precision("auto")
    assert (l1 - l0) - (l2 - l1) >= 2                     # the ordering kernels ran in the first call only
    assert torch.equal(grouped, plain)


def test_conv_is_deterministic_and_linear(cuda):
    from ss_conv import _ext
    from ss_conv.utils import synthetic as S
    ind = S.surface_voxels(range(8), 64, 16384, base_seed=50)
    outids, pairs, num = gpu_rulebook(ind, 8, [64] * 3, 3, 2, 1, 1, False, cuda)
    g = torch.Generator(device="cpu").manual_seed(0)
    a = torch.randn(ind.shape[0], 64, generator=g).to(cuda)
    b = torch.randn(ind.shape[0], 64, generator=g).to(cuda)
    W = (torch.randn(3, 3, 3, 64, 76, generator=g) / 40).to(cuda)
    _ext.set_precision("tf32")
    try:
        ya = _ext.indice_conv_fp32(a, W, pairs, num, outids.shape[0], 0, 0)
        ya2 = _ext.indice_conv_fp32(a, W, pairs, num, outids.shape[0], 0, 0)
        yb = _ext.indice_conv_fp32(b, W, pairs, num, outids.shape[0], 0, 0)
        yab = _ext.indice_conv_fp32(a + b, W, pairs, num, outids.shape[0], 0, 0)
        _ext.set_precision("fp32")
        yf = _ext.indice_conv_fp32(a, W, pairs, num, outids.shape[0], 0, 0)
    finally:
        _ext.set_precision("auto")
    _ext.check_status(cuda)
    assert torch.equal(ya, ya2)                                   # no atomics: bitwise repeatable
    scale = float(yf.abs().max())
    assert float((ya + yb - yab).abs().max()) <= 3e-3 * scale     # linear up to operand rounding
    assert float((ya - yf).abs().max()) <= 1e-3 * scale           # tensor-core vs exact path


def test_materialize_and_pack(cuda, golden):
    """Materialisation kernel vs the reference's einsum result for the golden layer."""
    from ss_conv.utils.kernel import SE3Kernel
    Rs_in = [tuple(int(v) for v in r) for r in golden["meta_Rs_in"]]
    Rs_out = [tuple(int(v) for v in r) for r in golden["meta_Rs_out"]]
    k = SE3Kernel(Rs_in, Rs_out, 3)
    state = {"weight": torch.from_numpy(golden["conv_weight"])}
    for i in range(len(Rs_out)):
        for j in range(len(Rs_in)):
            b = golden["basis_%d_%d" % (i, j)]
            if b.size:
                state["kernel_%d_%d" % (i, j)] = torch.from_numpy(b)
    k.load_state_dict(state)
    k.to(cuda)
    flt = k.filters().detach().cpu().numpy()
    assert flt.shape == golden["conv_filters"].shape
    assert np.abs(flt - golden["conv_filters"]).max() <= 1e-6
    W = k().detach().cpu().numpy()                                          # [Cout, Cin, k, k, k] view
    assert np.abs(W - np.transpose(golden["conv_filters"], (4, 3, 0, 1, 2))).max() <= 1e-6


def test_wide_submanifold_k5_stress(cuda):
    """The wide, high-order stress shape (256 -> 256 channels, kernel 5, submanifold, ~10 %
    random occupancy): oracle parity at reduced size, and at full size (batch 16, 48^3) sampled
    output rows against a direct float64 evaluation of their neighbourhoods."""
    from ss_conv import _ext
    from ss_conv.utils import synthetic as S
    rng = np.random.RandomState(4)
    small = S.bernoulli_voxels(range(2), 14, 0.1, base_seed=3)
    y, ref = _run(cuda, small, 2, 14, 5, 1, 2, True, 256, 256, "tf32")
    assert rel_err(y, ref) <= TOL["tf32"]
    ind = S.bernoulli_voxels(range(16), 48, 0.10, base_seed=40)
    n = ind.shape[0]
    g = torch.Generator(device="cpu").manual_seed(1)
    feats = torch.randn(n, 256, generator=g).to(cuda)
    W = (torch.randn(5, 5, 5, 256, 256, generator=g) / 180).to(cuda)
    outids, pairs, num = gpu_rulebook(ind, 16, [48] * 3, 5, 1, 2, 1, True, cuda)
    assert int(num[62]) == n and abs(float(num.sum()) / n - 12.5) < 1.0      # ~12.5 neighbours per voxel
    _ext.set_precision("tf32")
    try:
        y = _ext.indice_conv_fp32(feats, W, pairs, num, n, 0, 1)
        y2 = _ext.indice_conv_fp32(feats, W, pairs, num, n, 0, 1)
    finally:
        _ext.set_precision("auto")
    _ext.check_status(cuda)
    assert float((y - y2).abs().max() / y.abs().max()) <= 5e-5     # pair-list kernel: sums arrive in no fixed order
    nbr = _ext.neighbour_table(pairs, num, n)
    rows = torch.from_numpy(rng.choice(n, 64, replace=False)).to(cuda)
    src = nbr[:, rows]                                                      # [125, 64]
    gathered = feats.double()[src.clamp(min=0).long()] * (src >= 0).unsqueeze(-1)
    direct = torch.einsum("kri,kio->ro", gathered, W.double().reshape(125, 256, 256))
    err = float((y[rows].double() - direct).abs().max() / direct.abs().max())
    assert err <= TOL["tf32"]
    # 'auto' takes the pair-list kernel for this shape; the call above was it.  The output-stationary
    # kernel on the same operands differs only in the order of the fp32 sums.
    assert _ext._use_pairs(125, 256, 256, n, _ext.PREC_TF32)
    flt = W.reshape(125, 256, 256)
    y_rows = _ext.conv_forward(feats, flt, nbr, n, "tf32", algo="rows")
    assert float((y - y_rows).abs().max() / y_rows.abs().max()) <= 5e-5
    for prec in ("fp16", "bf16"):
        y16 = _ext.conv_forward(feats, flt, nbr, n, prec, algo="pairs")
        _ext.check_status(cuda)
        err = float((y16[rows].double() - direct).abs().max() / direct.abs().max())
        assert err <= TOL[prec]


@pytest.mark.parametrize("c_in,c_out,k,subm,batch,grid,per", [(64, 76, 3, False, 3, 14, 900), (32, 38, 3, True, 3, 14, 900),
                                                              (20, 8, 3, False, 3, 14, 900), (130, 270, 3, False, 2, 12, 330),
                                                              (3, 36, 3, True, 2, 12, 330), (16, 16, 5, True, 3, 14, 900),
                                                              (64, 76, 3, True, 4, 40, 20000), (200, 64, 2, False, 2, 16, 2000)])
def test_conv_fp16_operands(cuda, c_in, c_out, k, subm, batch, grid, per):
    """precision 'fp16': feature rows and filters rounded to fp16 (64 channels per 128-byte operand
    row), fp32 accumulation.  Odd channel counts exercise the zero padding of rows and slabs."""
    rng = np.random.RandomState(c_in * 3 + c_out)
    ind = random_voxels(rng, batch, grid, per)
    y, ref = _run(cuda, ind, batch, grid, k, 1 if subm else 2, k // 2 if subm else 0, subm, c_in, c_out, "fp16")
    assert rel_err(y, ref) <= TOL["fp16"]


def test_conv_half_entry_points(cuda):
    """indice_conv_half / indice_conv_backward_half (half tensors in and out) against the fp64
    oracle run on the same fp16-rounded inputs: only the final rounding to fp16 is left."""
    from ss_conv import _ext
    rng = np.random.RandomState(5)
    ind = random_voxels(rng, 2, 12, 500)
    c_in, c_out, k = 32, 48, 3
    feats = rng.randn(ind.shape[0], c_in).astype(np.float16)
    W = (rng.randn(k, k, k, c_in, c_out) / np.sqrt(c_in * k ** 3)).astype(np.float16)
    outids, pairs, num = gpu_rulebook(ind, 2, [12] * 3, k, 1, 1, 1, True, cuda)
    n_out = outids.shape[0]
    y = _ext.indice_conv_half(dev(feats, cuda), dev(W, cuda), pairs, num, n_out, 0, 1)
    assert y.dtype == torch.half
    ref = O.indice_conv_f64(feats.astype(np.float32), W.astype(np.float32), pairs.cpu().numpy(), num.cpu().numpy(), n_out)
    assert rel_err(y.float().cpu().numpy(), ref) <= 1e-3
    g = rng.randn(n_out, c_out).astype(np.float16)
    d_in, d_w = _ext.indice_conv_backward_half(dev(feats, cuda), dev(W, cuda), dev(g, cuda), pairs, num, 0, 1)
    torch.cuda.synchronize()
    _ext.check_status(cuda)
    assert d_in.dtype == torch.half and d_w.dtype == torch.half and d_w.shape == W.shape
    ref_in, ref_w = O.indice_conv_backward(feats.astype(np.float64), W.astype(np.float64), g.astype(np.float64),
                                           pairs.cpu().numpy(), num.cpu().numpy(), subm=True, dtype=np.float64)
    assert rel_err(d_in.float().cpu().numpy(), ref_in) <= 1e-3
    assert rel_err(d_w.float().cpu().numpy().reshape(ref_w.shape), ref_w) <= 2e-3


@pytest.mark.parametrize("c_in,c_out", [(64, 76), (3, 36), (30, 20)])
def test_conv_staged_rows_give_the_same_bits(cuda, monkeypatch, c_in, c_out):
    """Rounding the feature rows to TF32 once in a staging buffer (rows zero-padded to a multiple of
    four channels), or after every gather, feeds the tensor core the same operands: the results
    are bit-identical."""
    from ss_conv import _ext
    rng = np.random.RandomState(77)
    ind = random_voxels(rng, 4, 16, 2500)
    monkeypatch.setattr(_ext, "STAGING_MIN_ROWS", 1 << 30)
    plain, _ = _run(cuda, ind, 4, 16, 3, 1, 1, True, c_in, c_out, "tf32")
    monkeypatch.setattr(_ext, "STAGING_MIN_ROWS", 0)
    staged, ref = _run(cuda, ind, 4, 16, 3, 1, 1, True, c_in, c_out, "tf32")
    assert ind.shape[0] >= 64 * 128                # large enough for the library to stage
    np.testing.assert_array_equal(plain, staged)
    assert rel_err(staged, ref) <= TOL["tf32"]


@pytest.mark.parametrize("c_in,c_out,k,subm,batch,grid,per", [(64, 76, 3, False, 3, 14, 900), (130, 270, 3, False, 2, 12, 330),
                                                              (3, 36, 3, True, 2, 12, 330), (200, 64, 2, False, 2, 16, 2000)])
def test_conv_bf16_operands(cuda, c_in, c_out, k, subm, batch, grid, per):
    """precision 'bf16': feature rows and filters rounded to bfloat16 (fp32's range, 8 significant
    bits), fp32 accumulation; tolerance 1e-2 (the stated bf16 target)."""
    rng = np.random.RandomState(c_in * 3 + c_out)
    ind = random_voxels(rng, batch, grid, per)
    y, ref = _run(cuda, ind, batch, grid, k, 1 if subm else 2, k // 2 if subm else 0, subm, c_in, c_out, "bf16")
    assert rel_err(y, ref) <= TOL["bf16"]
    assert rel_err(y, ref) > 1e-5                 # really rounded to 8 bits, not silently the fp32 path


PAIR_SHAPES = [(64, 76, 3, False, 3, 14, 900),       # small filter matrix: two CTAs per SM, one strip each
               (32, 38, 3, True, 3, 14, 900),
               (30, 72, 3, False, 3, 14, 900),        # channel count not a multiple of four / of a slab
               (130, 270, 3, False, 2, 12, 330),      # two N tiles, more than one range of output channels
               (256, 256, 3, True, 3, 14, 900),       # TF32: the filter matrix needs two ranges; 16-bit: one
               (20, 16, 5, True, 3, 14, 900),         # 125 offsets, most lists shorter than a tile
               (64, 76, 3, True, 4, 40, 20000),       # several tiles per strip, strips of several CTAs per offset
               (256, 128, 5, True, 2, 24, 1400)]


@pytest.mark.parametrize("precision", ["tf32", "fp16", "bf16"])
@pytest.mark.parametrize("c_in,c_out,k,subm,batch,grid,per", PAIR_SHAPES)
def test_conv_pair_list_kernel(cuda, precision, c_in, c_out, k, subm, batch, grid, per):
    """The pair-list kernel (dense 128-pair tiles per kernel offset, filters resident in shared
    memory, reductions into the output rows) against the float64 oracle, and against the
    output-stationary kernel on the same operands (same products, another summation order)."""
    from ss_conv import _ext
    rng = np.random.RandomState(c_in + 7 * c_out + k)
    ind = random_voxels(rng, batch, grid, per)
    _ext.set_algo("pairs")
    try:
        assert _ext._use_pairs(k ** 3, c_in, c_out, 1 << 20, _ext._PREC_OF[precision])
        y, ref = _run(cuda, ind, batch, grid, k, 1 if subm else 2, k // 2 if subm else 1, subm, c_in, c_out, precision)
        y2, _ = _run(cuda, ind, batch, grid, k, 1 if subm else 2, k // 2 if subm else 1, subm, c_in, c_out, precision)
    finally:
        _ext.set_algo("auto")
    _ext.set_algo("rows")
    try:
        base, _ = _run(cuda, ind, batch, grid, k, 1 if subm else 2, k // 2 if subm else 1, subm, c_in, c_out, precision)
    finally:
        _ext.set_algo("auto")
    assert rel_err(y, ref) <= TOL[precision]
    assert rel_err(y, base) <= 5e-5                # identical operands, fp32 sums in another order
    assert rel_err(y2, y) <= 5e-5                  # a second call on the same (cached) lists


def test_conv_pair_list_kernel_empty_offsets_and_tiny_inputs(cuda):
    """Offsets without a single pair, lists shorter than one tile, one active voxel."""
    from ss_conv import _ext
    _ext.set_algo("pairs")
    try:
        for n in (1, 2, 130):
            ind = np.zeros((n, 4), dtype=np.int32)
            ind[:, 3] = np.arange(n) % 12
            ind[:, 2] = np.arange(n) // 12
            y, ref = _run(cuda, ind, 1, 12, 3, 1, 1, True, 32, 32, "tf32")
            assert rel_err(y, ref) <= TOL["tf32"]
    finally:
        _ext.set_algo("auto")


def _sampled_rows_check(cuda, feats, W, nbr, n_out, y, tol, rng, rows=96):
    """Sampled output rows of a full-size layer against a direct float64 evaluation of their
    neighbourhoods (the float64 oracle of the whole layer would take minutes on the CPU)."""
    K, ci, co = W.shape
    pick = torch.from_numpy(rng.choice(n_out, min(rows, n_out), replace=False)).to(cuda)
    src = nbr[:, pick]                                                       # [K, rows]
    gathered = feats.double()[src.clamp(min=0).long()] * (src >= 0).unsqueeze(-1)
    direct = torch.einsum("kri,kio->ro", gathered, W.double())
    err = float((y[pick].double() - direct).abs().max() / direct.abs().max())
    assert err <= tol, err
    return err


def test_cfg2_full_size_sampled_rows_against_float64(cuda):
    """The headline layer at benchmark size (batch 32, 64^3, 16384 surface points per sample, 64 -> 76
    channels, k3 s2 p1): sampled output rows of the TF32, bf16 and exact-fp32 paths against float64, and
    the rulebook's closed-form properties on the same batch."""
    from ss_conv import _ext
    from ss_conv.utils import synthetic as S
    rng = np.random.RandomState(8)
    ind = S.surface_voxels(range(32), 64, 16384, base_seed=1000)
    n = ind.shape[0]
    g = torch.Generator(device="cpu").manual_seed(2)
    feats = torch.randn(n, 64, generator=g).to(cuda)
    W = (torch.randn(27, 64, 76, generator=g) / 41.6).to(cuda)
    outids, pairs, num = gpu_rulebook(ind, 32, [64] * 3, 3, 2, 1, 1, False, cuda)
    n_out = outids.shape[0]
    nbr = _ext.neighbour_table(pairs, num, n_out)
    assert int((nbr >= 0).sum()) == int(num.sum())
    for prec in ("tf32", "bf16", "fp32"):
        y = _ext.conv_forward(feats, W, nbr, n_out, prec)
        _ext.check_status(cuda)
        _sampled_rows_check(cuda, feats, W, nbr, n_out, y, TOL[prec], rng)


def test_cfg3_stages_batch64_sampled_rows_against_float64(cuda):
    """The four strided stages of the backbone configuration at batch 64 (1024 points per object on a
    32^3 grid): geometry chained stage to stage, channel counts of the stages, sampled rows against
    float64 for every stage (the narrow first stage takes the exact fp32 kernel under 'auto')."""
    from ss_conv import _ext
    from ss_conv.sp_ops.ops import get_indice_pairs
    from ss_conv.utils import synthetic as S
    rng = np.random.RandomState(9)
    pts, _, ids = S.object_points(range(64), 1024, base_seed=7000)
    cells = np.floor((pts + 0.5) * 32).astype(np.int64)
    vox = np.unique(np.concatenate([ids[:, None], cells], 1), axis=0).astype(np.int32)
    cur = torch.from_numpy(vox).to(cuda)
    chans = [3, 30 + 6, 60 + 12, 120 + 24, 240 + 48]       # stage outputs carry their gate scalars
    cin = [3, 30, 60, 120]
    V = 32
    g = torch.Generator(device="cpu").manual_seed(3)
    for st in range(4):
        outids, pairs, num = get_indice_pairs(cur, 64, [V] * 3, 3, 2, 1, 1, 0, False, False)
        n_in, n_out = cur.shape[0], outids.shape[0]
        nbr = _ext.neighbour_table(pairs, num, n_out)
        feats = torch.randn(n_in, cin[st], generator=g).to(cuda)
        W = (torch.randn(27, cin[st], chans[st + 1], generator=g) / float(np.sqrt(27 * cin[st]))).to(cuda)
        for prec in ("auto", "tf32") if cin[st] >= 16 else ("auto",):
            y = _ext.conv_forward(feats, W, nbr, n_out, prec)
            _ext.check_status(cuda)
            tol = TOL["fp32"] if (prec == "auto" and cin[st] < 16) else TOL["tf32"]
            _sampled_rows_check(cuda, feats, W, nbr, n_out, y, tol, rng)
        cur, V = outids.contiguous(), V // 2
    assert V == 2 and cur.shape[0] <= 64 * 8


def test_conv1x1_through_the_gather_kernel(cuda):
    """A 1 x 1 x 1 convolution is the gather-GEMM with one offset and the identity table: it runs
    through the library's own kernels (no library GEMM on the path)."""
    from ss_conv import _ext
    from ss_conv.sp_ops.conv import SparseConvolution
    from ss_conv.sp_ops.tensor import SparseTensor
    rng = np.random.RandomState(12)
    ind = random_voxels(rng, 2, 12, 700)
    feats = rng.randn(ind.shape[0], 48).astype(np.float32)
    conv = SparseConvolution(3, 48, 40, 1, bias=False).to(cuda)
    assert conv.conv1x1
    with torch.no_grad():
        conv.weight.copy_(torch.randn_like(conv.weight) / 7)
    l0 = _ext.kernel_launches()
    _ext.set_precision("fp32")
    try:
        with torch.no_grad():
            y = conv(SparseTensor(dev(feats, cuda), dev(ind, cuda), [12] * 3, 2)).features.cpu().numpy()
    finally:
        _ext.set_precision("auto")
    assert _ext.kernel_launches() > l0               # the library's kernel ran
    ref = feats.astype(np.float64) @ conv.weight.detach().cpu().numpy().reshape(48, 40).astype(np.float64)
    assert rel_err(y, ref) <= TOL["fp32"]


@pytest.mark.parametrize("c_in,c_out,k,stride,subm", [(3, 36, 3, 2, False), (4, 38, 3, 1, False), (7, 20, 3, 1, True),
                                                      (16, 76, 3, 2, False), (13, 24, 5, 1, True), (1, 16, 3, 1, False)])
def test_conv_with_few_input_channels_packs_several_offsets_per_step(cuda, c_in, c_out, k, stride, subm):
    """TF32 layers whose padded input rows are 4, 8 or 16 floats pack the neighbours at 8, 4 or 2 kernel
    offsets side by side into one operand row (a 3-channel first layer runs 4 steps per tile instead of
    27).  Checked against the float64 oracle and the exact fp32 CUDA-core kernel at the TF32 tolerance
    (max rel err <= 1e-3), and for bit-repeatability."""
    from ss_conv import _ext
    rng = np.random.RandomState(100 + c_in)
    ind = random_voxels(rng, 3, 16, 1500)
    feats = rng.randn(ind.shape[0], c_in).astype(np.float32)
    W = (rng.randn(k ** 3, c_in, c_out) / np.sqrt(c_in * k ** 3)).astype(np.float32)
    pad = k // 2 if (subm or stride == 1) else 1
    outids, pairs, num = gpu_rulebook(ind, 3, [16] * 3, k, stride, pad, 1, subm, cuda)
    n_out = outids.shape[0]
    nbr = _ext.neighbour_table(pairs, num, n_out)
    f, w = dev(feats, cuda), dev(W, cuda)
    assert (_ext.lib().ssc_conv_packed_bytes(k ** 3, c_in, c_out, _ext.PREC_TF32)
            < k ** 3 * 128 * ((c_out + 15) // 16 * 16)) == (((c_in + 3) // 4 * 4) in (4, 8, 16))
    y = _ext.conv_forward(f, w, nbr, n_out, "tf32")
    y2 = _ext.conv_forward(f, w, nbr, n_out, "tf32")
    torch.cuda.synchronize()
    _ext.check_status(cuda)
    assert torch.equal(y, y2)
    ref = O.indice_conv_f64(feats, W, pairs.cpu().numpy(), num.cpu().numpy(), n_out)
    assert rel_err(y.cpu().numpy(), ref) <= 1e-3
    exact = _ext.conv_forward(f, w, nbr, n_out, "fp32")
    assert rel_err(y.cpu().numpy(), exact.cpu().numpy()) <= 1e-3


@pytest.mark.parametrize("ksize,s,p,subm,precision", [((3, 3, 3), 2, 1, False, "tf32"), ((3, 3, 3), 1, 1, True, "tf32"),
                                                      ((2, 2, 2), 2, 0, False, "fp16"), ((3, 2, 3), 1, 1, False, "tf32")])
def test_plane_order_of_a_forward_table(cuda, ksize, s, p, subm, precision):
    """ssc_nbr_row_order_planes: a permutation grouped by the kernel planes a row's neighbours lie in
    (groups that allow more offsets first, then ascending key, ascending rows inside a group), and the
    table moved into that order; with a device-side row count the rows beyond it come last; the
    convolution run through either gives the same bits as without."""
    from ss_conv import _ext
    rng = np.random.RandomState(sum(ksize) * 7 + s)
    ind = random_voxels(rng, 3, 24, 3000)
    outids, pairs, num = gpu_rulebook(ind, 3, [24] * 3, list(ksize), [s] * 3, [p, 0 if ksize[1] == 2 else p, p], [1] * 3, subm, cuda)
    n_in, n_out = ind.shape[0], outids.shape[0]
    nbr = _ext.neighbour_table(pairs, num, n_out)
    order, moved = _ext.nbr_row_order_planes(nbr, ksize, with_table=True)
    torch.cuda.synchronize()
    o, t = order.cpu().numpy(), nbr.cpu().numpy()
    has = (t >= 0).reshape(ksize + (n_out,))
    kx, ky, kz = ksize
    px = np.stack([has[x].any((0, 1)) for x in range(kx)])
    py = np.stack([has[:, y].any((0, 1)) for y in range(ky)])
    pz = np.stack([has[:, :, z].any((0, 1)) for z in range(kz)])
    key = np.zeros(n_out, np.int64)
    for i, plane in enumerate(list(px) + list(py) + list(pz)):
        key |= plane.astype(np.int64) << i
    weight = px.sum(0) * py.sum(0) * pz.sum(0)           # offsets the planes of a row allow
    want = np.lexsort((np.arange(n_out), key, -weight))
    assert np.array_equal(o, want)
    assert np.array_equal(moved.cpu().numpy(), t[:, o])
    # a capacity-sized table with the row count on the device: live rows first, in the same order
    live = n_out - 777
    n_dev = torch.tensor([live], dtype=torch.int32, device=cuda)
    o2 = _ext.nbr_row_order_planes(nbr, ksize, n_dev).cpu().numpy()
    assert np.array_equal(np.sort(o2), np.arange(n_out))
    assert np.array_equal(o2[:live], np.lexsort((np.arange(live), key[:live], -weight[:live])))
    assert np.array_equal(o2[live:], np.arange(live, n_out))
    c_in, c_out = 24, 40
    f = torch.randn(n_in, c_in, device=cuda)
    flt = torch.randn(kx * ky * kz, c_in, c_out, device=cuda) / 30
    plain = _ext.conv_forward(f, flt, nbr, n_out, precision, algo="rows")
    ordered = _ext.conv_forward(f, flt, nbr, n_out, precision, row_order=order, algo="rows")
    through_moved = _ext.conv_forward(f, flt, moved, n_out, precision, row_order=order, algo="rows", table_in_order=True)
    torch.cuda.synchronize()
    _ext.check_status(cuda)
    assert torch.equal(plain, ordered) and torch.equal(plain, through_moved)
