"""Backward kernels vs the reference's own CPU outputs (golden fixtures) and the oracle.
Tolerances as for the forward pass: exact-fp32 2e-5, TF32 operands 1e-3 (max|diff|/max|ref|
against the float64 evaluation); pool gradients are bit-exact (same accumulation order)."""
import numpy as np
import pytest
import torch

import ssconv_oracle as O
from gpu_helpers import dev, gpu_rulebook, random_voxels, rel_err

pytestmark = pytest.mark.gpu
TOL = {"fp32": 2e-5, "tf32": 1e-3}


@pytest.mark.parametrize("k,s,p,subm,precision", [(3, 2, 1, False, "tf32"), (3, 1, 1, True, "tf32"), (2, 2, 0, False, "fp16"),
                                                  (5, 2, 2, False, "tf32")])
def test_row_order_is_a_grouping_permutation_and_changes_no_bit(cuda, k, s, p, subm, precision):
    """ssc_nbr_row_order: a permutation, groups = first used offset in ascending order, ascending
    rows inside a group; the convolution run through it gives the same bits as without."""
    from ss_conv import _ext
    rng = np.random.RandomState(k * 11 + s)
    ind = random_voxels(rng, 3, 24, 4000)
    outids, pairs, num = gpu_rulebook(ind, 3, [24] * 3, k, s, p, 1, subm, cuda)
    n_in, n_out = ind.shape[0], outids.shape[0]
    nbr = _ext.neighbour_table(pairs, num, n_out)
    nbr_in = _ext.input_major_table(nbr, n_in)
    order = _ext.nbr_row_order(nbr_in)
    torch.cuda.synchronize()
    o = order.cpu().numpy()
    t = nbr_in.cpu().numpy()
    assert np.array_equal(np.sort(o), np.arange(n_in))
    has = t >= 0
    key = np.where(has.any(0), has.argmax(0), t.shape[0])
    want = np.lexsort((np.arange(n_in), key))       # by key, then by row number
    assert np.array_equal(o, want)
    c_out, c_in = 40, 24
    g = torch.randn(n_out, c_out, device=cuda)
    fT = torch.randn(k ** 3, c_out, c_in, device=cuda) / 30
    plain = _ext.conv_forward(g, fT, nbr_in, n_in, precision)
    ordered = _ext.conv_forward(g, fT, nbr_in, n_in, precision, row_order=order)
    torch.cuda.synchronize()
    _ext.check_status(cuda)
    assert torch.equal(plain, ordered)


def test_conv_backward_recorded_with_parallel_branches(cuda):
    """conv_backward recorded into a CUDA graph puts the filter gradient on a side stream (a
    parallel branch of the graph); the replay gives the bits of the eager call."""
    from ss_conv import _ext
    rng = np.random.RandomState(21)
    ind = random_voxels(rng, 3, 24, 4000)
    outids, pairs, num = gpu_rulebook(ind, 3, [24] * 3, 3, 2, 1, 1, False, cuda)
    n_in, n_out = ind.shape[0], outids.shape[0]
    nbr = _ext.neighbour_table(pairs, num, n_out)
    f = torch.randn(n_in, 32, device=cuda)
    g = torch.randn(n_out, 40, device=cuda)
    flt = torch.randn(27, 32, 40, device=cuda) / 30
    want_in, want_w = _ext.conv_backward(f, flt, g, nbr, precision="tf32")
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got_in, got_w = _ext.conv_backward(f, flt, g, nbr, precision="tf32")
    got_in.zero_()
    got_w.zero_()
    graph.replay()
    torch.cuda.synchronize()
    _ext.check_status(cuda)
    assert torch.equal(got_in, want_in) and torch.equal(got_w, want_w)


@pytest.mark.parametrize("tag", ["bw_strided", "bw_subm"])
def test_conv_backward_matches_reference_outputs(cuda, golden, tag):
    from ss_conv import _ext
    subm = int(golden[tag + "_geom"][3])
    _ext.set_precision("fp32")
    try:
        d_in, d_flt = _ext.indice_conv_backward_fp32(dev(golden[tag + "_features"], cuda), dev(golden[tag + "_filters"], cuda),
                                                     dev(golden[tag + "_dout"], cuda), dev(golden[tag + "_pairs"], cuda),
                                                     dev(golden[tag + "_num"], cuda), 0, subm)
        torch.cuda.synchronize()
        _ext.check_status(cuda)
    finally:
        _ext.set_precision("auto")
    assert d_flt.shape == golden[tag + "_filters"].shape
    assert rel_err(d_in.cpu().numpy(), golden[tag + "_din"]) <= TOL["fp32"]
    assert rel_err(d_flt.cpu().numpy(), golden[tag + "_dfilters"]) <= TOL["fp32"]


@pytest.mark.parametrize("precision", ["fp32", "tf32"])
@pytest.mark.parametrize("c_in,c_out,k,s,p,subm", [(32, 38, 3, 2, 1, False), (64, 76, 3, 1, 1, True), (20, 70, 2, 2, 0, False),
                                                     (130, 40, 3, 1, 1, False)])
def test_conv_backward_vs_float64_oracle(cuda, precision, c_in, c_out, k, s, p, subm):
    from ss_conv import _ext
    rng = np.random.RandomState(c_in + 7 * c_out)
    ind = random_voxels(rng, 2, 12, 400)
    outids, pairs, num = gpu_rulebook(ind, 2, [12] * 3, k, s, p, 1, subm, cuda)
    n_out = outids.shape[0]
    feats = rng.randn(ind.shape[0], c_in).astype(np.float32)
    W = (rng.randn(k, k, k, c_in, c_out) / np.sqrt(c_in * k ** 3)).astype(np.float32)
    dout = rng.randn(n_out, c_out).astype(np.float32)
    _ext.set_precision(precision)
    try:
        d_in, d_flt = _ext.indice_conv_backward_fp32(dev(feats, cuda), dev(W, cuda), dev(dout, cuda), pairs, num, 0, int(subm))
        again = _ext.indice_conv_backward_fp32(dev(feats, cuda), dev(W, cuda), dev(dout, cuda), pairs, num, 0, int(subm))
        torch.cuda.synchronize()
        _ext.check_status(cuda)
    finally:
        _ext.set_precision("auto")
    ref_in, ref_flt = O.indice_conv_backward(feats, W, dout, pairs.cpu().numpy(), num.cpu().numpy(), False, False,
                                             dtype=np.float64)
    assert rel_err(d_in.cpu().numpy(), ref_in) <= TOL[precision]
    assert rel_err(d_flt.cpu().numpy().reshape(ref_flt.shape), ref_flt) <= TOL[precision]
    assert torch.equal(d_in, again[0]) and torch.equal(d_flt, again[1])                        # bitwise repeatable


def test_pool_backward_bit_exact(cuda, golden):
    from ss_conv import _ext
    pairs, num = dev(golden["bw_strided_pairs"], cuda), dev(golden["bw_strided_num"], cuda)
    d = _ext.indice_maxpool_backward_fp32(dev(golden["bw_pool_features"], cuda), dev(golden["bw_pool_out"], cuda),
                                          dev(golden["bw_pool_dout"], cuda), pairs, num)
    np.testing.assert_array_equal(d.cpu().numpy(), golden["bw_pool_din"])
    # average pool: divisor = kernel volume (use_gs) and = number of present inputs
    n_out = golden["bw_pool_out"].shape[0]
    for rf in (None, O.summary_rf(golden["bw_strided_pairs"], golden["bw_strided_num"], n_out)):
        want = O.indice_avgpool_backward(golden["bw_pool_features"], golden["bw_pool_dout"], golden["bw_strided_pairs"],
                                         golden["bw_strided_num"], np.full(n_out, 27, np.int32) if rf is None else rf)
        got = _ext.indice_avgpool_backward_fp32(dev(golden["bw_pool_features"], cuda), dev(golden["bw_pool_out"], cuda),
                                                dev(golden["bw_pool_dout"], cuda), pairs, num,
                                                None if rf is None else dev(rf, cuda))
        np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_global_pool_backward(cuda):
    from ss_conv.sp_ops.functional import global_avgpool, global_maxpool
    rng = np.random.RandomState(5)
    offsets = np.array([0, 7, 7, 40, 100], dtype=np.int32)      # one empty sample
    feats = rng.randn(100, 37).astype(np.float32)
    g = rng.randn(4, 37).astype(np.float32)
    for fn, name in ((global_avgpool, "avg"), (global_maxpool, "max")):
        x = dev(feats, cuda).requires_grad_(True)
        y = fn(x, dev(offsets, cuda))
        y.backward(dev(g, cuda))
        if name == "avg":
            want = O.global_avgpool_backward(g, offsets, 100)
        else:
            _, maxidx = O.global_maxpool(feats, offsets)
            want = O.global_maxpool_backward(g, maxidx, 100)
        np.testing.assert_allclose(x.grad.cpu().numpy(), want, rtol=1e-6, atol=1e-7)


def test_training_step_through_a_steerable_layer(cuda):
    """loss.backward() through Convolution (training mode) + MaxPool: gradients reach the input
    features and the steerable weights; the weight gradient passes the adjoint identity
    <M v, G> = <v, M^T G> of the linear materialisation, and the feature gradient matches the
    oracle evaluated with the layer's own filters."""
    from ss_conv import _ext
    from ss_conv.convolution import Convolution
    from ss_conv.pool import MaxPool
    from ss_conv.sp_ops.tensor import SparseTensor
    torch.manual_seed(12)
    rng = np.random.RandomState(12)
    conv = Convolution([(2, 0), (2, 1)], [(3, 0), (1, 1), (1, 2)], 3, stride=2, padding=1).to(cuda).train()
    pool = MaxPool(2, stride=2)
    ind = random_voxels(rng, 2, 12, 300)
    feats = rng.randn(ind.shape[0], conv.in_channels).astype(np.float32)
    _ext.set_precision("fp32")
    try:
        x = dev(feats, cuda).requires_grad_(True)
        y = pool(conv(SparseTensor(x, dev(ind, cuda), [12] * 3, 2)))
        G = torch.randn_like(y.features)
        (y.features * G).sum().backward()
        torch.cuda.synchronize()
        assert x.grad is not None and conv.kernel.weight.grad is not None
        # oracle chain with the layer's filters
        W = conv.kernel.filters().detach().cpu().numpy()
        o1, p1, n1 = O.get_indice_pairs(ind, 2, [12] * 3, 3, 2, 1, 1, False)
        y1 = O.indice_conv(feats, W, p1, n1, o1.shape[0])
        o2, p2, n2 = O.get_indice_pairs(o1, 2, [6] * 3, 2, 2, 0, 1, False)
        y2 = O.indice_maxpool(y1, p2, n2, o2.shape[0])
        # row orders: GPU ascending flat index, oracle first-seen -> compare through canonical order
        perm1 = np.lexsort((o1[:, 3], o1[:, 2], o1[:, 1], o1[:, 0]))
        perm2 = np.lexsort((o2[:, 3], o2[:, 2], o2[:, 1], o2[:, 0]))
        Gn = np.zeros_like(y2)
        Gn[perm2] = G.cpu().numpy()
        d1 = O.indice_maxpool_backward(y1, y2, Gn, p2, n2)
        d_x, d_W = O.indice_conv_backward(feats, W, d1, p1, n1, False, False, dtype=np.float64)
        assert rel_err(x.grad.cpu().numpy(), d_x) <= 1e-4
        # adjoint identity for the weights
        v = torch.randn_like(conv.kernel.weight)
        Mv = conv.kernel.filters(v.detach()).detach().cpu().numpy().astype(np.float64).reshape(d_W.shape)
        lhs = float((Mv * d_W).sum())
        rhs = float((v.double() * conv.kernel.weight.grad.double()).sum())
        assert abs(lhs - rhs) <= 1e-4 * max(1.0, abs(lhs))
        assert perm1.shape[0] == o1.shape[0]
    finally:
        _ext.set_precision("auto")


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
def test_voxelizer_gradients(cuda, mode):
    """voxelize_bp on explicit rule rows vs the oracle, and the gradient the fused Point2Voxel
    attaches to its voxel features vs the same oracle on the equivalent rule rows."""
    from ss_conv import _ext
    from ss_conv.sp_ops.voxelize import Point2Voxel
    from ss_conv.utils import synthetic as S
    rng = np.random.RandomState(mode)
    pts, fts, ids = S.object_points(range(3), 400, base_seed=30)
    p2v = Point2Voxel([8] * 3, [1.0 / 8] * 3, mode)
    x = dev(fts, cuda).requires_grad_(True)
    _, sp, _, _ = p2v(dev(pts, cuda), x, dev(ids, cuda))
    G = rng.randn(*sp.features.shape).astype(np.float32)
    sp.features.backward(dev(G, cuda))
    # equivalent rule rows from the oracle's voxelizer on the same points
    kept, _, vox, _, inverse = O.point2voxel(pts, fts, ids, [8] * 3, [1.0 / 8] * 3, mode)
    assert kept.shape[0] == pts.shape[0]                       # every synthetic point is in range
    np.testing.assert_array_equal(vox, sp.indices.cpu().numpy())
    max_active = 1 if mode in (1, 2) else int(np.bincount(inverse).max())
    maps = O.voxel2point_map(inverse, vox.shape[0], max_active, mode)
    want = O.voxelize_bp(G, maps, mode, pts.shape[0])
    np.testing.assert_allclose(x.grad.cpu().numpy(), want, rtol=1e-6, atol=1e-7)
    d_feats = torch.empty((pts.shape[0], fts.shape[1]), dtype=torch.float32, device=cuda)
    _ext.voxelize_bp(dev(G, cuda), d_feats, dev(maps.astype(np.int32), cuda), mode, vox.shape[0], max_active, fts.shape[1])
    np.testing.assert_allclose(d_feats.cpu().numpy(), want, rtol=1e-6, atol=1e-7)


def test_interpolation_gradient(cuda):
    from ss_conv.sp_ops.functional import three_interpolate
    rng = np.random.RandomState(3)
    m, n, c = 50, 400, 9
    feats = rng.randn(m, c).astype(np.float32)
    idx = rng.randint(0, m, size=(n, 3)).astype(np.int32)
    w = rng.rand(n, 3).astype(np.float32)
    w /= w.sum(1, keepdims=True)
    g = rng.randn(n, c).astype(np.float32)
    x = dev(feats, cuda).requires_grad_(True)
    y = three_interpolate(x, dev(idx, cuda), dev(w, cuda))
    y.backward(dev(g, cuda))
    want = O.three_interpolate_bp(g, idx, w, m)
    assert rel_err(x.grad.cpu().numpy(), want) <= 1e-5


def test_training_step_through_conv_bn_gate(cuda):
    """One optimiser-style step through Convolution -> BatchNorm(train) -> gated Activation ->
    GlobalAvgPool: every parameter receives a finite, non-zero gradient, the running statistics
    move, and the differentiable composite equals the fused inference path in eval mode."""
    from ss_conv import _ext
    from ss_conv.activation import Activation
    from ss_conv.batchnorm import BatchNorm
    from ss_conv.convolution import Convolution
    from ss_conv.pool import GlobalAvgPool
    from ss_conv.sp_ops.tensor import SparseTensor
    torch.manual_seed(2)
    rng = np.random.RandomState(2)
    Rs_in, Rs_mid = [(3, 0)], [(4, 0), (2, 1), (1, 2)]
    gated = Rs_mid + [(3, 0)]
    conv = Convolution(Rs_in, gated, 3, stride=2, padding=1).to(cuda)
    bn = BatchNorm(gated).to(cuda)
    act = Activation(Rs_mid, (torch.relu, torch.sigmoid), bias=True, checkpoint=False).to(cuda)
    gp = GlobalAvgPool()
    ind = random_voxels(rng, 3, 10, 200)
    feats = dev(rng.randn(ind.shape[0], 3).astype(np.float32), cuda)
    _ext.set_precision("fp32")
    try:
        for m in (conv, bn, act):
            m.train()
        rv0 = bn.running_var.clone()
        y = gp(act(bn(conv(SparseTensor(feats, dev(ind, cuda), [10] * 3, 3)))))
        y.pow(2).sum().backward()
        params = [conv.kernel.weight, bn.weight, bn.bias] + list(act.parameters())
        for p in params:
            assert p.grad is not None and torch.isfinite(p.grad).all() and float(p.grad.abs().sum()) > 0
        assert not torch.equal(rv0, bn.running_var)
        for m in (conv, bn, act):
            m.eval()
        x1 = act(bn(conv(SparseTensor(feats, dev(ind, cuda), [10] * 3, 3)))).features        # composite (grad on)
        with torch.no_grad():
            x2 = act(bn(conv(SparseTensor(feats, dev(ind, cuda), [10] * 3, 3)))).features    # fused kernels
        assert rel_err(x1.detach().cpu().numpy(), x2.cpu().numpy()) <= 1e-5
    finally:
        _ext.set_precision("auto")


@pytest.mark.parametrize("training", [True, False])
def test_batchnorm_and_gate_backward_kernels(cuda, training):
    """BatchNorm and the gated activation under autograd run the library's kernels in both
    directions (ssc_bn_stats / ssc_bn_bwd / ssc_gate_bwd).  Gradients of the input and of the affine
    parameters, the outputs and the updated running statistics against the same layers evaluated as a
    float64 composite of torch ops on the CPU (what the reference's autograd would compute,
    SS_Conv_lib/ss_conv/batchnorm.py:49-136, activation.py:55-100)."""
    import copy
    from ss_conv import _ext
    from ss_conv.activation import Activation
    from ss_conv.batchnorm import BatchNorm
    from ss_conv.sp_ops.tensor import SparseTensor
    torch.manual_seed(4)
    Rs = [(3, 0), (2, 1), (2, 2), (1, 3)]
    gated = Rs + [(5, 0)]
    n, c = 3000, 3 + 6 + 10 + 7 + 5
    bn = BatchNorm(gated, momentum=0.1).to(cuda)
    act = Activation(Rs, (torch.relu, torch.sigmoid), bias=False, checkpoint=False).to(cuda)
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.normal_(0, 0.3)
        bn.running_var.uniform_(0.5, 2.0)
        bn.running_mean.normal_(0, 0.2)
    bn.train(training)
    bn64, act64 = copy.deepcopy(bn).double().cpu(), copy.deepcopy(act).double().cpu()
    x = (torch.randn(n, c, device=cuda) * 1.3 + 0.2).requires_grad_(True)
    coef = torch.randn(n, 26, device=cuda)
    ind = torch.zeros(n, 4, dtype=torch.int32, device=cuda)
    l0 = _ext.kernel_launches()
    y = act(bn(SparseTensor(x, ind, [8] * 3, 1))).features
    (y * coef).sum().backward()
    assert _ext.kernel_launches() - l0 >= 6          # statistics, affine pass, gate, and their backward kernels
    x64 = x.detach().double().cpu().requires_grad_(True)
    y64 = act64._gate_composite(bn64._differentiable(x64))
    (y64 * coef.double().cpu()).sum().backward()
    assert rel_err(y.detach().cpu().numpy(), y64.detach().numpy()) <= 2e-5
    assert rel_err(x.grad.cpu().numpy(), x64.grad.numpy()) <= 1e-4
    assert rel_err(bn.weight.grad.cpu().numpy(), bn64.weight.grad.numpy()) <= 1e-4
    assert rel_err(bn.bias.grad.cpu().numpy(), bn64.bias.grad.numpy()) <= 1e-4
    assert rel_err(bn.running_var.cpu().numpy(), bn64.running_var.numpy()) <= 1e-5
    assert rel_err(bn.running_mean.cpu().numpy(), bn64.running_mean.numpy()) <= 1e-5
    if training:      # the batch statistics are added in a fixed order: a second pass gives the same bits
        bn2 = copy.deepcopy(bn)
        x2 = x.detach().clone().requires_grad_(True)
        ya = bn(SparseTensor(x2, ind, [8] * 3, 1)).features
        yb = bn2(SparseTensor(x2, ind, [8] * 3, 1)).features
        assert torch.equal(ya, yb)
