"""The CPU oracle against arrays produced by running the reference itself
(tests/golden/make_golden.py): rulebooks bit-exact including order, floating point within
the tolerance written at each check."""
import numpy as np
import pytest

import ssconv_oracle as O


def test_rulebook_matches_reference_cpu_functor(golden):
    ind = golden["rb_indices"]
    for ci, (k, s, p, d, subm) in enumerate(golden["rb_cases"]):
        outids, pairs, num = O.get_indice_pairs(ind, 2, [12] * 3, int(k), int(s), int(p), int(d), bool(subm))
        assert np.array_equal(outids, golden["rb%d_outids" % ci])
        assert np.array_equal(num, golden["rb%d_num" % ci])
        assert np.array_equal(pairs, golden["rb%d_pairs" % ci])


def test_rulebook_edge_cases():
    empty = np.zeros((0, 4), np.int32)
    outids, pairs, num = O.get_indice_pairs(empty, 1, [8] * 3, 3, 1, 1, 1, False)
    assert outids.shape == (0, 4) and pairs.shape == (27, 2, 0) and num.sum() == 0
    one = np.array([[0, 0, 0, 0]], np.int32)
    outids, pairs, num = O.get_indice_pairs(one, 1, [4] * 3, 3, 1, 1, 1, False)
    assert outids.shape[0] == 8 and num.sum() == 8
    outids, pairs, num = O.get_indice_pairs(one, 1, [4] * 3, 3, 1, 1, 1, True)
    assert num.sum() == 1 and num[13] == 1 and pairs[13, 0, 0] == 0 and pairs[13, 1, 0] == 0


def _layer(golden, tag, subm=False, **kw):
    ind, feats = golden[tag + "_indices"], golden[tag + "_features"]
    outids, pairs, num = O.get_indice_pairs(ind, 2, [10] * 3, subm=subm, **kw)
    y = O.indice_conv(feats, golden[tag + "_filters"], pairs, num, outids.shape[0], False, subm)
    assert np.array_equal(outids, golden[tag + "_out_indices"])
    ref = golden[tag + "_out_features"]
    assert np.abs(y - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())


def test_layer_outputs_match_reference(golden):
    _layer(golden, "conv", ksize=3, stride=1, padding=1)
    _layer(golden, "strided", ksize=3, stride=2, padding=1)
    _layer(golden, "subm", subm=True, ksize=3, padding=1)


def _bases(golden, Rs_in, Rs_out):
    b = {}
    for i in range(len(Rs_out)):
        for j in range(len(Rs_in)):
            a = golden["basis_%d_%d" % (i, j)]
            b[(i, j)] = None if a.size == 0 else a
    return b


def test_materialisation_matches_reference(golden):
    Rs_in = [tuple(r) for r in golden["meta_Rs_in"]]
    Rs_out = [tuple(r) for r in golden["meta_Rs_out"]]
    W = O.combination(golden["conv_weight"], _bases(golden, Rs_in, Rs_out), Rs_in, Rs_out, 3)
    flt = O.filters_from_kernel(W)
    assert flt.shape == golden["conv_filters"].shape
    assert np.abs(flt - golden["conv_filters"]).max() <= 1e-6


def test_batchnorm_and_activation_match_reference(golden):
    Rs_out = [tuple(r) for r in golden["meta_Rs_out"]]
    x = golden["conv_out_features"]
    rm, rv, w, b = (golden["bn_" + n] for n in ("running_mean", "running_var", "weight", "bias"))
    y = O.batchnorm_eval(x, Rs_out, rm, rv, w, b)
    assert np.abs(y - golden["bn_eval_out"]).max() <= 2e-6 * max(1.0, np.abs(y).max())
    yt, nm, nv = O.batchnorm_train(x, Rs_out, rm, rv, w, b, momentum=0.1)
    assert np.abs(yt - golden["bn_train_out"]).max() <= 1e-5 * max(1.0, np.abs(yt).max())
    assert np.allclose(nm, golden["bn_train_running_mean"], rtol=1e-5, atol=1e-6)
    assert np.allclose(nv, golden["bn_train_running_var"], rtol=1e-5, atol=1e-6)
    z = O.gated_activation(golden["bn_eval_out"], Rs_out[:-1], "relu", "sigmoid", golden["act_scalar_bias"],
                           golden["act_gate_bias"])
    assert np.abs(z - golden["act_out"]).max() <= 2e-6


def test_maxpool_matches_reference(golden):
    ind = golden["conv_out_indices"]
    outids, pairs, num = O.get_indice_pairs(ind, 2, [10] * 3, 2, 2, 0, 1, False)
    y = O.indice_maxpool(golden["conv_out_features"], pairs, num, outids.shape[0])
    assert np.array_equal(outids, golden["maxpool_out_indices"])
    assert np.array_equal(y, golden["maxpool_out_features"])


def test_sparse_conv_equals_dense_conv3d():
    """Invariant the reference satisfies: sparse conv == dense cross-correlation on the
    densified input, read at the active outputs."""
    import torch
    rng = np.random.RandomState(3)
    V, B, Cin, Cout = 8, 2, 5, 7
    flat = rng.choice(V ** 3 * B, 150, replace=False)
    ind = np.stack([flat // V ** 3, (flat // (V * V)) % V, (flat // V) % V, flat % V], 1).astype(np.int32)
    feats = rng.randn(ind.shape[0], Cin).astype(np.float32)
    W = rng.randn(3, 3, 3, Cin, Cout).astype(np.float32)
    outids, pairs, num = O.get_indice_pairs(ind, B, [V] * 3, 3, 1, 1, 1, False)
    y = O.indice_conv(feats, W, pairs, num, outids.shape[0])
    dense = torch.zeros(B, Cin, V, V, V)
    dense[ind[:, 0], :, ind[:, 1], ind[:, 2], ind[:, 3]] = torch.from_numpy(feats)
    out = torch.nn.functional.conv3d(dense, torch.from_numpy(W).permute(4, 3, 0, 1, 2), padding=1)
    got = out[outids[:, 0], :, outids[:, 1], outids[:, 2], outids[:, 3]].numpy()
    assert np.abs(got - y).max() <= 1e-4


def test_helpers_small_cases():
    feats = np.arange(12, dtype=np.float32).reshape(6, 2)
    off = np.array([0, 2, 2, 6], np.int32)
    avg = O.global_avgpool(feats, off)
    assert np.allclose(avg[0], [1, 2]) and np.isnan(avg[1]).all() and np.allclose(avg[2], [7, 8])
    mx, arg = O.global_maxpool(feats, off)
    assert np.allclose(mx[2], [10, 11]) and arg[2, 0] == 5 and arg[1, 0] == -1
    inv = np.array([0, 1, 0, 2, 1, 0], np.int32)
    maps = O.voxel2point_map(inv, 3, 3, 4)
    assert maps[0].tolist() == [3, 0, 2, 5] and maps[2].tolist()[:2] == [1, 3]
    assert O.voxel2point_map(inv, 3, 1, 1)[:, 1].tolist() == [0, 1, 3]
    assert O.voxel2point_map(inv, 3, 1, 2)[:, 1].tolist() == [5, 4, 3]
    vf = O.voxelize_fp(feats, maps, 4)
    assert np.allclose(vf[0], feats[[0, 2, 5]].mean(0))
    unknown = np.array([[0, 0, 0, 0], [1, 1, 1, 1]], np.float32)
    known = np.array([[0, 1, 0, 0], [0, 0, 2, 0], [1, 1, 1, 1], [0, 0, 0, 3], [0, 5, 5, 5]], np.float32)
    d2, idx = O.three_nn(unknown, known)
    assert idx[0].tolist() == [0, 1, 3] and d2[0].tolist() == [1, 4, 9]
    assert idx[1].tolist() == [2, 0, 0] and np.isinf(d2[1, 1])


def test_transposed_rulebook_matches_reference(golden):
    """Transposed geometry: compared in canonical order (the oracle does not reproduce the
    reference's first-seen output numbering for this case)."""
    ind = golden["rbt_indices"]
    for ci, (k, s, p, op) in enumerate(golden["rbt_cases"]):
        got = O.get_indice_pairs(ind, 2, [8] * 3, int(k), int(s), int(p), 1, False, True, int(op))
        ref = (golden["rbt%d_outids" % ci], golden["rbt%d_pairs" % ci], golden["rbt%d_num" % ci])
        a, b = O.canonical_rulebook(*got), O.canonical_rulebook(*ref)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[2], b[2])
        for x, y in zip(a[1], b[1]):
            assert np.array_equal(x, y)


@pytest.mark.parametrize("tag", ["bw_strided", "bw_subm"])
def test_conv_backward_matches_reference(golden, tag):
    """indiceConvBackward<float> of the compiled reference (CPU) vs the restatement."""
    k, s, p, subm = (int(v) for v in golden[tag + "_geom"])
    d_in, d_flt = O.indice_conv_backward(golden[tag + "_features"], golden[tag + "_filters"], golden[tag + "_dout"],
                                         golden[tag + "_pairs"], golden[tag + "_num"], False, bool(subm))
    ref_in, ref_flt = golden[tag + "_din"], golden[tag + "_dfilters"].reshape(d_flt.shape)
    assert np.abs(d_in - ref_in).max() <= 2e-6 * max(1.0, np.abs(ref_in).max())
    assert np.abs(d_flt - ref_flt).max() <= 2e-6 * max(1.0, np.abs(ref_flt).max())
    # and the rulebook the fixture was made with is the one the oracle builds
    o, pr, nm = O.get_indice_pairs(golden["bw_indices"], 2, [10] * 3, k, s, p, 1, bool(subm))
    np.testing.assert_array_equal(nm, golden[tag + "_num"])


def test_maxpool_backward_matches_reference(golden):
    d = O.indice_maxpool_backward(golden["bw_pool_features"], golden["bw_pool_out"], golden["bw_pool_dout"],
                                  golden["bw_strided_pairs"], golden["bw_strided_num"])
    np.testing.assert_array_equal(d, golden["bw_pool_din"])
    y = O.indice_maxpool(golden["bw_pool_features"], golden["bw_strided_pairs"], golden["bw_strided_num"],
                         golden["bw_pool_out"].shape[0])
    np.testing.assert_array_equal(y, golden["bw_pool_out"])


def test_feature_steering_matches_reference(golden):
    """Point / feature change of frame of Feature_Steering_Module and the representation matrices
    of rotation_utils.D_from_matrix (reference outputs) vs the restatement and this package's
    own Wigner-D construction (no constants file)."""
    import sys
    import os
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", "ss-conv_b200"))
    from ss_conv.utils import SO3
    irrep = [int(v) for v in golden["fsm_irrep"]]
    R, t, s, ids = golden["fsm_R"], golden["fsm_t"], golden["fsm_s"], golden["fsm_ids"]
    d_ref = [golden["fsm_D%d" % l] for l in range(len(irrep))]
    for l in range(len(irrep)):
        assert np.abs(SO3.D_from_matrix(R.astype(np.float64), l) - d_ref[l]).max() <= 1e-6     # R is stored in fp32
    assert np.abs(O.steer_points(golden["fsm_points"], ids, R, t, s) - golden["fsm_new_points"]).max() <= 2e-6
    assert np.abs(O.steer_points(golden["fsm_points"], ids, R, t) - golden["fsm_new_points_noscale"]).max() <= 2e-6
    assert np.abs(O.steer_feats(golden["fsm_feats"], ids, d_ref, irrep) - golden["fsm_new_feats"]).max() <= 5e-6
