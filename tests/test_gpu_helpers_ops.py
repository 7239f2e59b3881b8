"""Pooling, voxelization, interpolation and BN/activation kernels vs the oracle."""
import numpy as np
import pytest
import torch

import ssconv_oracle as O
from gpu_helpers import dev, gpu_rulebook, random_voxels, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("c", [64, 30, 3])
def test_max_and_avg_pool(cuda, c):
    from ss_conv import _ext
    rng = np.random.RandomState(c)
    ind = random_voxels(rng, 3, 12, 400)
    feats = rng.randn(ind.shape[0], c).astype(np.float32)
    for k, s, p in ((2, 2, 0), (3, 2, 1)):
        outids, pairs, num = gpu_rulebook(ind, 3, [12] * 3, k, s, p, 1, False, cuda)
        pn, nn = pairs.cpu().numpy(), num.cpu().numpy()
        n_out = outids.shape[0]
        mx = _ext.indice_maxpool_fp32(dev(feats, cuda), pairs, num, n_out).cpu().numpy()
        assert np.array_equal(mx, O.indice_maxpool(feats, pn, nn, n_out))          # bit-exact
        av = _ext.indice_avgpool_fp32(dev(feats, cuda), pairs, num, n_out, None).cpu().numpy()
        assert np.array_equal(av, O.indice_avgpool(feats, pn, nn, n_out))          # same order, bit-exact
        rf = _ext.indiceSummaryRF(pairs, num, n_out)
        assert np.array_equal(rf.cpu().numpy(), O.summary_rf(pn, nn, n_out))
        av2 = _ext.indice_avgpool_fp32(dev(feats, cuda), pairs, num, n_out, rf).cpu().numpy()
        assert np.array_equal(av2, O.indice_avgpool(feats, pn, nn, n_out, O.summary_rf(pn, nn, n_out)))


def test_pool_modules_and_golden(cuda, golden):
    from ss_conv.pool import MaxPool, AvgPool
    from ss_conv.sp_ops.tensor import SparseTensor
    x = SparseTensor(dev(golden["conv_out_features"], cuda), dev(golden["conv_out_indices"], cuda), [10] * 3, 2)
    z = MaxPool(2, stride=2)(x)
    zi = z.indices.cpu().numpy()
    perm = O.renumber_rows(golden["maxpool_out_indices"])
    assert np.array_equal(zi, golden["maxpool_out_indices"][perm])
    assert np.array_equal(z.features.cpu().numpy(), golden["maxpool_out_features"][perm])
    a = AvgPool(3, stride=2, padding=1)(x)
    assert a.features.shape[0] == a.indices.shape[0] and a.spatial_shape == [5, 5, 5]


def test_global_pools(cuda):
    from ss_conv.pool import GlobalAvgPool, GlobalMaxPool
    from ss_conv.sp_ops.tensor import SparseTensor
    rng = np.random.RandomState(0)
    counts = [37, 1, 200, 64, 9]
    ind = np.concatenate([np.stack([np.full(n, b), np.arange(n) % 16, np.arange(n) // 16, np.zeros(n)], 1)
                          for b, n in enumerate(counts)]).astype(np.int32)
    feats = rng.randn(ind.shape[0], 70).astype(np.float32)
    x = SparseTensor(dev(feats, cuda), dev(ind, cuda), [16] * 3, 5)
    off = x.get_offsets()
    assert off.cpu().tolist() == np.concatenate([[0], np.cumsum(counts)]).tolist()
    avg = GlobalAvgPool()(x).cpu().numpy()
    ref = O.global_avgpool(feats, off.cpu().numpy())
    assert np.abs(avg - ref).max() <= 1e-5          # pairwise instead of sequential summation
    mx = GlobalMaxPool()(x.features, off).cpu().numpy()
    rmx, rarg = O.global_maxpool(feats, off.cpu().numpy())
    assert np.array_equal(mx, rmx)
    from ss_conv import _ext
    out = torch.zeros(5, 70, device=cuda)
    arg = torch.zeros(5, 70, dtype=torch.int32, device=cuda)
    _ext.global_maxpool_fp(x.features, off, out, arg, 5, 70)
    assert np.array_equal(arg.cpu().numpy(), rarg)
    # empty sample: mean is NaN (0/0), max is -inf with arg -1, as in the reference kernels
    off2 = torch.tensor([0, 3, 3, 5], dtype=torch.int32, device=cuda)
    a2 = GlobalAvgPool()(x.features[:5].contiguous(), off2).cpu().numpy()
    assert np.isnan(a2[1]).all() and np.isfinite(a2[0]).all()


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
def test_voxel2point_map_and_voxelize(cuda, mode):
    from ss_conv.sp_ops.functional import voxel2point_mapping, voxelization
    rng = np.random.RandomState(mode)
    n, m = 500, 90
    inverse = rng.randint(0, m, n).astype(np.int32)
    inverse[:m] = np.arange(m)
    counts = np.bincount(inverse, minlength=m)
    max_active = 1 if mode in (1, 2) else int(counts.max())
    feats = rng.rand(n, 5).astype(np.float32)
    maps = voxel2point_mapping(dev(inverse, cuda), m, max_active, mode)
    ref_maps = O.voxel2point_map(inverse, m, max_active, mode)
    assert np.array_equal(maps.cpu().numpy(), ref_maps)
    out = voxelization(dev(feats, cuda), maps, mode).cpu().numpy()
    assert np.array_equal(out, O.voxelize_fp(feats, ref_maps, mode))


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
def test_point2voxel_module(cuda, mode):
    from ss_conv.sp_ops.voxelize import Point2Voxel
    from ss_conv.utils import synthetic as S
    pts, fts, ids = S.object_points(range(4), 700, base_seed=9)
    pts[5] = [0.7, 0.0, 0.0]                        # out of range: dropped
    V = 16
    p2v = Point2Voxel([V] * 3, [1.0 / V] * 3, mode)
    vp, sp, vids, flag = p2v(dev(pts, cuda), dev(fts, cuda), dev(ids, cuda))
    rp, rfeat, rocc, rids, rinv = O.point2voxel(pts, fts, ids, [V] * 3, [1.0 / V] * 3, mode)
    assert np.array_equal(vp.cpu().numpy(), rp) and np.array_equal(vids.cpu().numpy(), rids)
    assert np.array_equal(sp.indices.cpu().numpy(), rocc)
    assert np.array_equal(sp.features.cpu().numpy(), rfeat)
    assert flag.cpu().tolist() == [1.0] * 4 and sp.batch_size == 4


def test_point2voxel_empty_sample(cuda):
    from ss_conv.sp_ops.voxelize import Point2Voxel
    rng = np.random.RandomState(0)
    pts = rng.uniform(-0.4, 0.4, (300, 3)).astype(np.float32)
    ids = np.repeat(np.arange(3), 100)
    pts[100:200] = 5.0                              # sample 1 loses every point
    p2v = Point2Voxel([8] * 3, [0.125] * 3, 4)
    vp, sp, vids, flag = p2v(dev(pts, cuda), dev(pts, cuda), dev(ids, cuda))
    assert flag.cpu().tolist() == [1.0, 0.0, 1.0]
    assert vp.shape[0] == 201 and int((vids == 1).sum()) == 1
    row = sp.indices.cpu().numpy()
    assert (row[row[:, 0] == 1][:, 1:] == 4).all()   # the injected zero point sits in the centre cell


def test_three_nn_and_interpolate(cuda):
    from ss_conv.sp_ops.voxelize import Voxel2Point, Point2Voxel
    from ss_conv.sp_ops.functional import three_nn
    from ss_conv.utils import synthetic as S
    pts, fts, ids = S.object_points(range(3), 900, base_seed=3)
    V = 16
    p2v = Point2Voxel([V] * 3, [1.0 / V] * 3, 4)
    vp, sp, vids, _ = p2v(dev(pts, cuda), dev(fts, cuda), dev(ids, cuda))
    sp.features = torch.randn(sp.features.shape[0], 19, device=cuda)
    v2p = Voxel2Point(unit_voxel_extent=[1.0 / V] * 3)
    out = v2p(sp, vp, vids).cpu().numpy()
    ref, d2, idx = O.voxel2point(sp.features.cpu().numpy(), sp.indices.cpu().numpy(), [V] * 3, [1.0 / V] * 3,
                                 vp.cpu().numpy(), vids.cpu().numpy())
    centres, _ = v2p._get_vertice_feats(sp)
    unknown = torch.cat([vids.float().unsqueeze(1), vp], 1)
    gd, gi = three_nn(unknown, centres)
    assert np.array_equal(gi.cpu().numpy(), idx)                    # same neighbours, same tie order
    assert np.array_equal((gd ** 2).cpu().numpy().round(6), d2.round(6)) or np.allclose(gd.cpu().numpy() ** 2, d2, rtol=1e-6)
    assert np.abs(out - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())
    # a sample with fewer than three voxels keeps +inf distances and index 0
    unknown2 = torch.tensor([[7.0, 0, 0, 0]], device=cuda)
    known2 = torch.tensor([[7.0, 1, 0, 0], [3.0, 0, 0, 0]], device=cuda)
    d, i = three_nn(unknown2, known2)
    assert i.cpu().tolist() == [[0, 0, 0]] and torch.isinf(d[0, 1]) and float(d[0, 0]) == 1.0


def test_batchnorm_activation_golden(cuda, golden):
    from ss_conv.batchnorm import BatchNorm
    from ss_conv.activation import Activation
    from ss_conv.sp_ops.tensor import SparseTensor
    Rs_out = [tuple(int(v) for v in r) for r in golden["meta_Rs_out"]]
    bn = BatchNorm(Rs_out, momentum=0.1).to(cuda)
    with torch.no_grad():
        for n in ("running_mean", "running_var", "weight", "bias"):
            getattr(bn, n).copy_(dev(golden["bn_" + n], cuda))
    x = dev(golden["conv_out_features"], cuda)
    ind = dev(golden["conv_out_indices"], cuda)
    bn.eval()
    y = bn(SparseTensor(x.clone(), ind, [10] * 3, 2)).features.cpu().numpy()
    assert np.abs(y - golden["bn_eval_out"]).max() <= 3e-6 * max(1.0, np.abs(y).max())
    bn.train()
    stats0 = (bn.running_mean.clone(), bn.running_var.clone())
    for fused in (True, False):          # statistics kernels (no autograd) / differentiable composite
        with torch.no_grad():
            bn.running_mean.copy_(stats0[0])
            bn.running_var.copy_(stats0[1])
        with torch.set_grad_enabled(not fused):
            yt = bn(SparseTensor(x.clone(), ind, [10] * 3, 2)).features.detach().cpu().numpy()
        assert np.abs(yt - golden["bn_train_out"]).max() <= 2e-5 * max(1.0, np.abs(yt).max())
        assert np.allclose(bn.running_mean.cpu().numpy(), golden["bn_train_running_mean"], rtol=1e-5, atol=1e-6)
        assert np.allclose(bn.running_var.cpu().numpy(), golden["bn_train_running_var"], rtol=1e-5, atol=1e-6)
    bn.eval()
    act = Activation(Rs_out[:-1], (torch.relu, torch.sigmoid), bias=True, checkpoint=False).to(cuda)
    with torch.no_grad():
        act.scalar_act.bias.copy_(dev(golden["act_scalar_bias"], cuda))
        act.gate_act.bias.copy_(dev(golden["act_gate_bias"], cuda))
    act.eval()
    z = act(SparseTensor(dev(golden["bn_eval_out"], cuda), ind, [10] * 3, 2)).features.cpu().numpy()
    assert z.shape == golden["act_out"].shape
    assert np.abs(z - golden["act_out"]).max() <= 3e-6
    # a non-fusable callable takes the composite path and agrees with the fused kernel
    act2 = Activation(Rs_out[:-1], (lambda v: torch.relu(v), torch.sigmoid), bias=True, checkpoint=False).to(cuda)
    act2.load_state_dict(act.state_dict())
    with torch.no_grad():
        z2 = act2(SparseTensor(dev(golden["bn_eval_out"], cuda), ind, [10] * 3, 2)).features.cpu().numpy()
    assert np.abs(z2 - z).max() <= 2e-6


def test_feature_steering_kernel_and_module(cuda, golden):
    """ssc_steer_fwd vs the reference's own outputs; then Feature_Steering_Module end to end with
    the identity pose = plain voxelize + two SS_Conv blocks."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", "ss-conv_b200"))
    from ss_conv_modules import Feature_Steering_Module, SS_Conv
    from ss_conv import _ext
    from ss_conv.sp_ops.tensor import SparseTensor
    irrep = tuple(int(v) for v in golden["fsm_irrep"])
    torch.manual_seed(5)
    fsm = Feature_Steering_Module(irrep, kernel_size=3, dropout_p=0.0, voxel_num_limit=[8] * 3,
                                  unit_voxel_extent=[0.25] * 3).to(cuda).eval()
    pts, fts = dev(golden["fsm_points"], cuda), dev(golden["fsm_feats"], cuda)
    ids = dev(golden["fsm_ids"], cuda)
    R, t, s = dev(golden["fsm_R"], cuda), dev(golden["fsm_t"], cuda), dev(golden["fsm_s"], cuda)
    new_p, new_f = fsm.steer(pts, fts, ids, R, t, s)
    assert np.abs(new_p.cpu().numpy() - golden["fsm_new_points"]).max() <= 2e-6
    assert np.abs(new_f.cpu().numpy() - golden["fsm_new_feats"]).max() <= 5e-6
    new_p2, _ = fsm.steer(pts, fts, ids, R, t)
    assert np.abs(new_p2.cpu().numpy() - golden["fsm_new_points_noscale"]).max() <= 2e-6
    # whole module, identity pose
    _ext.set_precision("fp32")
    try:
        with torch.no_grad():
            B = 3
            eye = torch.eye(3, device=cuda).repeat(B, 1, 1)
            zero = torch.zeros(B, 3, device=cuda)
            vp, vf, vi, flag = fsm(pts, fts, ids, eye, zero)
            assert isinstance(vf, SparseTensor) and float(flag.sum()) == B
            _, sp, _, _ = fsm.p2v(pts, fts, ids)
            want = fsm.conv2(fsm.conv1(sp))
            assert torch.equal(vf.indices, want.indices)
            assert rel_err(vf.features.cpu().numpy(), want.features.cpu().numpy()) <= 1e-5
            assert isinstance(fsm.conv1, SS_Conv)
        _ext.check_status(cuda)
    finally:
        _ext.set_precision("auto")


@pytest.mark.parametrize("axis", [0, 1, 2])
def test_steerable_convolution_is_equivariant_under_grid_rotations(cuda, axis):
    """Steering the input by a rotation that maps the voxel grid onto itself (90 degrees about a
    coordinate axis) and convolving equals convolving and steering the output, through
    convolution + batch norm + gated activation, when the features are rotated by the
    representation in the frame of the filter basis (frame="kernel")."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", "ss-conv_b200"))
    from ss_conv_modules import Feature_Steering_Module
    from ss_conv import _ext
    torch.manual_seed(11 + axis)
    rng = np.random.RandomState(11 + axis)
    irrep = (2, 2, 1)
    V, unit = 8, 0.25
    fsm = Feature_Steering_Module(irrep, kernel_size=3, dropout_p=0.0, voxel_num_limit=[V] * 3,
                                  unit_voxel_extent=[unit] * 3, voxelization_mode=4, frame="kernel").to(cuda).eval()
    with torch.no_grad():
        fsm.conv1.bn.running_var.uniform_(0.5, 1.5)
        fsm.conv1.bn.running_mean.normal_(0, 0.1)
    # one point per occupied voxel, at the voxel centre
    occ = np.argwhere(rng.rand(2, V, V, V) < 0.15)
    pts = ((occ[:, 1:] + 0.5) * unit - 0.5 * V * unit).astype(np.float32)
    ids = occ[:, 0].astype(np.int32)
    C = sum(m * (2 * l + 1) for l, m in enumerate(irrep))
    fts = rng.randn(pts.shape[0], C).astype(np.float32)
    c, s = 0.0, 1.0
    R1 = np.eye(3, dtype=np.float32)
    i, j = [(1, 2), (2, 0), (0, 1)][axis]
    R1[i, i], R1[i, j], R1[j, i], R1[j, j] = c, -s, s, c
    R = dev(np.stack([R1, R1]), cuda)
    zero = torch.zeros(2, 3, device=cuda)
    P, Fe, I = dev(pts, cuda), dev(fts, cuda), dev(ids, cuda)

    def centres(sp):
        return ((sp.indices[:, 1:].float() + 0.5) * unit - 0.5 * V * unit), sp.indices[:, 0].contiguous()

    def keyed(sp):
        k = ((sp.indices[:, 0] * V + sp.indices[:, 1]) * V + sp.indices[:, 2]) * V + sp.indices[:, 3]
        order = torch.argsort(k)
        return k[order].cpu().numpy(), sp.features[order].cpu().numpy()

    _ext.set_precision("fp32")
    try:
        with torch.no_grad():
            # A: steer, voxelize, convolve
            p1, f1 = fsm.steer(P, Fe, I, R, zero)
            a = fsm.conv1(fsm.p2v(p1, f1, I)[1])
            # B: voxelize, convolve, then steer the output voxels
            b0 = fsm.conv1(fsm.p2v(P, Fe, I)[1])
            cp, cid = centres(b0)
            order = torch.argsort(cid, stable=True)
            p2, f2 = fsm.steer(cp[order].contiguous(), b0.features[order].contiguous(), cid[order].contiguous(), R, zero)
            b = fsm.p2v(p2, f2, cid[order].contiguous())[1]
        ka, fa = keyed(a)
        kb, fb = keyed(b)
        np.testing.assert_array_equal(ka, kb)
        assert rel_err(fa, fb) <= 1e-4
    finally:
        _ext.set_precision("auto")


def test_half_precision_pool_entry_points(cuda):
    """indice_maxpool_half / indice_avgpool_half and their backward entry points (half tensors in and
    out, SS_Conv_lib/src/ss_conv_ops.h:58-63) against the fp32 entry points on the same fp16 values."""
    from ss_conv import _ext
    rng = np.random.RandomState(6)
    ind = random_voxels(rng, 2, 12, 500)
    outids, pairs, num = gpu_rulebook(ind, 2, [12] * 3, 2, 2, 0, 1, False, cuda)
    n_out = outids.shape[0]
    f16 = dev(rng.randn(ind.shape[0], 24).astype(np.float32), cuda).half()
    mx = _ext.indice_maxpool_half(f16, pairs, num, n_out)
    assert mx.dtype == torch.half and torch.equal(mx, _ext.indice_maxpool_fp32(f16.float(), pairs, num, n_out).half())
    av = _ext.indice_avgpool_half(f16, pairs, num, n_out, None)
    assert av.dtype == torch.half and torch.equal(av, _ext.indice_avgpool_fp32(f16.float(), pairs, num, n_out, None).half())
    g = torch.randn(n_out, 24, device=cuda).half()
    d1 = _ext.indice_maxpool_backward_half(f16, mx, g, pairs, num)
    assert d1.dtype == torch.half and d1.shape == f16.shape
    assert torch.equal(d1, _ext.indice_maxpool_backward_fp32(f16.float(), mx.float(), g.float(), pairs, num).half())
    d2 = _ext.indice_avgpool_backward_half(f16, av, g, pairs, num, None)
    assert d2.dtype == torch.half and d2.shape == f16.shape


def test_scatter_add_rate_kernel_adds_what_it_reports(cuda):
    """The reduction-only measurement kernel (ssc_scatter_add_rate): every list position adds 1.0 to
    a whole row, so the row sums must equal the occurrence counts of the rows it walked and the total
    must equal the bytes it reports (exact: small integers in fp32)."""
    from ss_conv import _ext
    rng = np.random.RandomState(9)
    n_rows, width = 3000, 64
    rows = torch.from_numpy(rng.randint(0, n_rows, 50000).astype(np.int32)).to(cuda)
    for lanes, warps in ((8, 16), (1, 16), (2, 4), (4, 1)):
        out = torch.zeros(n_rows, width, device=cuda)
        nbytes = _ext.scatter_add_rate(out, rows, 1, lanes, warps)
        torch.cuda.synchronize()
        _ext.check_status(cuda)
        positions = nbytes // (width * 4)
        assert positions % 32 == 0 and positions > 0
        idx = torch.arange(positions, device=cuda) % rows.numel()
        expect = torch.bincount(rows[idx].long(), minlength=n_rows).float()
        assert torch.equal(out, expect[:, None].expand(n_rows, width)), (lanes, warps)
