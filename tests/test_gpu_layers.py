"""Whole layers through the public ss_conv API vs the reference's own outputs (golden
fixtures) and the small backbone end to end."""
import numpy as np
import pytest
import torch

import ssconv_oracle as O
from gpu_helpers import dev, rel_err

pytestmark = pytest.mark.gpu


def _load_conv(golden, tag, cuda, **kw):
    from ss_conv.convolution import Convolution
    Rs_in = [tuple(int(v) for v in r) for r in golden["meta_Rs_in"]]
    Rs_out = [tuple(int(v) for v in r) for r in golden["meta_Rs_out"]]
    conv = Convolution(Rs_in, Rs_out, **kw).eval()
    state = {"kernel.weight": torch.from_numpy(golden[tag + "_weight"])}
    for i in range(len(Rs_out)):
        for j in range(len(Rs_in)):
            b = golden["basis_%d_%d" % (i, j)]
            if b.size:
                state["kernel.kernel_%d_%d" % (i, j)] = torch.from_numpy(b)
    conv.load_state_dict(state)
    return conv.to(cuda)


@pytest.mark.parametrize("precision,tol", [("fp32", 2e-5), ("tf32", 1e-3)])
@pytest.mark.parametrize("tag,kw", [("conv", dict(kernel_size=3, stride=1, padding=1)),
                                    ("strided", dict(kernel_size=3, stride=2, padding=1)),
                                    ("subm", dict(kernel_size=3, subm=True, padding=1))])
def test_convolution_layer_matches_reference_output(cuda, golden, tag, kw, precision, tol):
    from ss_conv import _ext
    from ss_conv.sp_ops.tensor import SparseTensor
    conv = _load_conv(golden, tag, cuda, **kw)
    x = SparseTensor(dev(golden[tag + "_features"], cuda), dev(golden[tag + "_indices"], cuda), [10] * 3, 2)
    _ext.set_precision(precision)
    try:
        with torch.no_grad():
            y = conv(x)
    finally:
        _ext.set_precision("auto")
    _ext.check_status(cuda)
    ref_idx = golden[tag + "_out_indices"]
    perm = O.renumber_rows(ref_idx)                 # reference CPU order -> ascending (b,x,y,z)
    if tag == "subm":
        assert np.array_equal(y.indices.cpu().numpy(), ref_idx)
        perm = np.arange(ref_idx.shape[0])
    else:
        assert np.array_equal(y.indices.cpu().numpy(), ref_idx[perm])
    assert rel_err(y.features.cpu().numpy(), golden[tag + "_out_features"][perm]) <= tol


def test_indice_key_reuse_and_state_dict_names(cuda, golden):
    from ss_conv.sp_ops.tensor import SparseTensor
    conv_a = _load_conv(golden, "subm", cuda, kernel_size=3, subm=True, padding=1, indice_key="k0")
    names = set(conv_a.state_dict().keys())
    assert "kernel.weight" in names and "kernel.kernel_0_0" in names
    x = SparseTensor(dev(golden["subm_features"], cuda), dev(golden["subm_indices"], cuda), [10] * 3, 2)
    with torch.no_grad():
        y1 = conv_a(x)
    assert "k0" in x.indice_dict and y1.indice_dict is x.indice_dict
    pairs_first = x.indice_dict["k0"][2]
    x2 = SparseTensor(x.features, x.indices, [10] * 3, 2)
    x2.indice_dict = x.indice_dict
    with torch.no_grad():
        y2 = conv_a(x2)
    assert x2.indice_dict["k0"][2] is pairs_first            # rulebook reused, not rebuilt
    assert torch.equal(y1.features, y2.features)


def test_backbone_forward_matches_oracle_chain(cuda):
    """Point2Voxel -> 2 x (Conv s2 + BN + gate) -> GlobalAvgPool, layer by layer against the
    oracle fed with the same parameters."""
    from ss_conv import _ext
    from ss_conv.convolution import Convolution
    from ss_conv.batchnorm import BatchNorm
    from ss_conv.activation import Activation
    from ss_conv.pool import GlobalAvgPool
    from ss_conv.sp_ops.voxelize import Point2Voxel
    from ss_conv.utils import synthetic as S
    torch.manual_seed(0)
    irreps = [(3,), (4, 2, 1), (6, 3, 2)]
    pts, fts, ids = S.object_points(range(4), 512, base_seed=21)
    V = 16
    x = Point2Voxel([V] * 3, [1.0 / V] * 3, 4)(dev(pts, cuda), dev(fts, cuda), dev(ids, cuda))[1]
    cur_idx, cur_feat, shape = x.indices.cpu().numpy(), x.features.cpu().numpy(), [V] * 3
    _ext.set_precision("fp32")
    try:
        for li in range(2):
            Rs_in = [(m, l) for l, m in enumerate(irreps[li])]
            Rs_act = [(m, l) for l, m in enumerate(irreps[li + 1])]
            Rs_out = Rs_act + [(sum(irreps[li + 1][1:]), 0)]
            conv = Convolution(Rs_in, Rs_out, 3, stride=2, padding=1).to(cuda).eval()
            bn = BatchNorm(Rs_out).to(cuda).eval()
            with torch.no_grad():
                bn.running_var.uniform_(0.5, 1.5)
                bn.running_mean.normal_(0, 0.1)
            act = Activation(Rs_act, (torch.relu, torch.sigmoid), bias=False, checkpoint=False)
            with torch.no_grad():
                x = act(bn(conv(x)))
            flt = conv.weight.cpu().numpy()
            outids, pairs, num = O.get_indice_pairs(cur_idx, 4, shape, 3, 2, 1, 1, False)
            perm = O.renumber_rows(outids)
            y = O.indice_conv(cur_feat, flt, pairs, num, outids.shape[0])[perm]
            y = O.batchnorm_eval(y, Rs_out, bn.running_mean.cpu().numpy(), bn.running_var.cpu().numpy(),
                                 bn.weight.detach().cpu().numpy(), bn.bias.detach().cpu().numpy())
            y = O.gated_activation(y, Rs_act, "relu", "sigmoid")
            shape = [s // 2 for s in shape]
            cur_idx, cur_feat = outids[perm], y
            assert np.array_equal(x.indices.cpu().numpy(), cur_idx)
            assert rel_err(x.features.cpu().numpy(), cur_feat) <= 5e-5
    finally:
        _ext.set_precision("auto")
    pooled = GlobalAvgPool()(x).cpu().numpy()
    counts = np.bincount(cur_idx[:, 0], minlength=4)
    ref = O.global_avgpool(cur_feat, np.concatenate([[0], np.cumsum(counts)]))
    assert rel_err(pooled, ref) <= 5e-5


def test_host_stream_gives_the_same_results_as_direct_calls(cuda):
    """Batches of different sizes fed from pinned host memory through the overlapped
    upload / compute / download pipeline come back in order and bit-equal to the results of
    calling the step directly on device tensors."""
    from ss_conv import _ext
    from ss_conv.pipeline import HostStream
    from ss_conv.pool import MaxPool
    from ss_conv.sp_ops.tensor import SparseTensor
    from ss_conv.utils import synthetic as S
    pool = MaxPool(2, stride=2)

    def step(f, i):
        y = pool(SparseTensor(f, i, [16] * 3, 2))
        return y.features, y.indices

    batches = []
    for r, n in enumerate((300, 120, 511, 64, 300)):
        ind = S.bernoulli_voxels(range(2), 16, n / (2 * 16 ** 3), base_seed=40 + 2 * r)
        feats = S.features(ind.shape[0], 5, 90 + r)
        batches.append((torch.from_numpy(feats).pin_memory(), torch.from_numpy(ind).pin_memory()))
    want = []
    for f, i in batches:
        of, oi = step(f.to(cuda), i.to(cuda))
        want.append((of.cpu().numpy(), oi.cpu().numpy()))
    feed = HostStream(step, cuda, max_rows=max(i.shape[0] for _, i in batches))
    got = [(of.numpy().copy(), oi.numpy().copy()) for of, oi in feed.run(iter(batches))]
    assert len(got) == len(want)
    for (gf, gi), (wf, wi) in zip(got, want):
        np.testing.assert_array_equal(gi, wi)
        np.testing.assert_array_equal(gf, wf)
    assert list(feed.run(iter([]))) == []
    _ext.check_status(cuda)


def test_layers_that_run_ahead_of_the_output_count(cuda, monkeypatch):
    """A strided convolution + max pool whose rulebooks are sized by a guessed capacity (output
    count read back after the kernels were queued) give bit-identical results to the exact
    path, also when the guess was too small and the layer has to be redone."""
    from ss_conv import _ext
    from ss_conv.pool import MaxPool
    from ss_conv.sp_ops.conv import SparseConvolution
    from ss_conv.sp_ops.tensor import SparseTensor
    from ss_conv.utils import synthetic as S
    torch.manual_seed(3)
    conv = SparseConvolution(3, 16, 24, 3, stride=2, padding=1, bias=True).to(cuda)
    pool = MaxPool(2, stride=2)
    ind = S.bernoulli_voxels(range(3), 20, 0.15, base_seed=11)
    feats = S.features(ind.shape[0], 16, 5)

    def run():
        with torch.no_grad():
            y = pool(conv(SparseTensor(dev(feats, cuda), dev(ind, cuda), [20] * 3, 3)))
        torch.cuda.synchronize()
        _ext.check_status(cuda)
        return y.features.cpu().numpy(), y.indices.cpu().numpy()

    _ext.set_precision("fp32")
    try:
        monkeypatch.setattr(_ext, "AHEAD", False)
        exact = run()
        monkeypatch.setattr(_ext, "AHEAD", True)
        _ext._ratio_hint.clear()
        first = run()                       # no hint yet: exact path, records the ratios
        assert len(_ext._ratio_hint) == 2
        l0 = _ext.kernel_launches()
        ahead = run()                       # capacities guessed from the recorded ratios
        n_ahead = _ext.kernel_launches() - l0
        for k in list(_ext._ratio_hint):
            _ext._ratio_hint[k] = 1e-3      # far too small: both layers overflow and are redone
        l0 = _ext.kernel_launches()
        redone = run()
        assert _ext.kernel_launches() - l0 > n_ahead
        again = run()                       # the overflow raised the hints again
    finally:
        _ext.set_precision("auto")
    for got in (first, ahead, redone, again):
        np.testing.assert_array_equal(got[1], exact[1])
        np.testing.assert_array_equal(got[0], exact[0])


def test_pending_row_counts_chain_through_a_network(cuda, monkeypatch):
    """conv -> BN -> gate -> conv -> BN -> gate -> max pool -> global pool with every row count left
    on the device until the end equals the same network run layer by layer with exact counts,
    also after a capacity overflow in the middle of the chain."""
    from ss_conv import _ext
    from ss_conv.activation import Activation
    from ss_conv.batchnorm import BatchNorm
    from ss_conv.convolution import Convolution
    from ss_conv.pool import GlobalAvgPool, MaxPool
    from ss_conv.sp_ops.tensor import SparseTensor
    from ss_conv.utils import synthetic as S
    torch.manual_seed(9)
    Rs = [[(2, 0), (1, 1)], [(4, 0), (2, 1)], [(4, 0), (2, 1), (1, 2)]]

    def gated(rs):
        return rs + [(sum(m for m, l in rs if l > 0), 0)]

    layers = []
    for a, b in zip(Rs[:-1], Rs[1:]):
        conv = Convolution(a, gated(b), 3, stride=2, padding=1).to(cuda).eval()
        bn = BatchNorm(gated(b)).to(cuda).eval()
        with torch.no_grad():
            bn.running_var.uniform_(0.5, 1.5)
            bn.running_mean.normal_(0, 0.1)
        layers.append((conv, bn, Activation(b, (torch.relu, torch.sigmoid), bias=False, checkpoint=False)))
    pool, gpool = MaxPool(2, stride=2), GlobalAvgPool()
    ind = S.bernoulli_voxels(range(4), 24, 0.2, base_seed=21)
    feats = S.features(ind.shape[0], 5, 8)

    def run(check_pending):
        with torch.no_grad():
            x = SparseTensor(dev(feats, cuda), dev(ind, cuda), [24] * 3, 4)
            for conv, bn, act in layers:
                x = act(bn(conv(x)))
            x = pool(x)
            assert x.pending() == check_pending
            pooled = gpool(x)
            assert not x.pending()
        torch.cuda.synchronize()
        _ext.check_status(cuda)
        return pooled.cpu().numpy(), x.features.cpu().numpy(), x.indices.cpu().numpy()

    _ext.set_precision("fp32")
    try:
        monkeypatch.setattr(_ext, "AHEAD", False)
        exact = run(False)
        monkeypatch.setattr(_ext, "AHEAD", True)
        _ext._ratio_hint.clear()
        first = run(False)                 # records the ratios layer by layer
        chained = run(True)
        keys = sorted(_ext._ratio_hint)
        _ext._ratio_hint[keys[1]] = 1e-3   # one layer in the middle will overflow
        overflowed = run(True)
        again = run(True)
    finally:
        _ext.set_precision("auto")
    for got in (first, chained, overflowed, again):
        for g, e in zip(got, exact):
            np.testing.assert_array_equal(g, e)


def test_graphed_chain_replays_match_eager_results(cuda):
    """conv -> BN -> gate -> max pool (-> global pool) recorded as one CUDA graph and replayed on
    batches of different sizes equals the eager exact results; a batch that overflows a capacity
    falls back to the exact path and the graph is recorded again."""
    from ss_conv import _ext
    from ss_conv.activation import Activation
    from ss_conv.batchnorm import BatchNorm
    from ss_conv.convolution import Convolution
    from ss_conv.graph import GraphedChain
    from ss_conv.pool import GlobalAvgPool, MaxPool
    from ss_conv.sp_ops.tensor import SparseTensor
    from ss_conv.utils import synthetic as S
    torch.manual_seed(4)
    Rs_in, Rs_out = [(2, 0), (1, 1)], [(4, 0), (2, 1)]
    gated = Rs_out + [(2, 0)]
    conv = Convolution(Rs_in, gated, 3, stride=2, padding=1).to(cuda).eval()
    bn = BatchNorm(gated).to(cuda).eval()
    act = Activation(Rs_out, (torch.relu, torch.sigmoid), bias=False, checkpoint=False)
    pool, gpool = MaxPool(2, stride=2), GlobalAvgPool()

    def sparse_net(x):
        return pool(act(bn(conv(x))))

    def dense_net(x):
        return gpool(sparse_net(x))

    batches = []
    for r, occ in enumerate((0.10, 0.06, 0.12, 0.10)):
        ind = S.bernoulli_voxels(range(3), 20, occ, base_seed=50 + 3 * r)
        batches.append((dev(S.features(ind.shape[0], 5, 60 + r), cuda), dev(ind, cuda)))
    cap = max(i.shape[0] for _, i in batches)
    _ext.set_precision("fp32")
    try:
        with torch.no_grad():
            want = []
            for f, i in batches:
                y = sparse_net(SparseTensor(f, i, [20] * 3, 3))
                want.append((y.features.clone(), y.indices.clone(), dense_net(SparseTensor(f, i, [20] * 3, 3)).clone()))
            g_sparse = GraphedChain(sparse_net, [20] * 3, 3, 5, cap, cuda)
            g_dense = GraphedChain(dense_net, [20] * 3, 3, 5, cap, cuda)
            for rep in range(2):
                for (f, i), (wf, wi, wd) in zip(batches, want):
                    y = g_sparse(f, i)
                    assert torch.equal(y.indices, wi) and torch.equal(y.features, wf)
                    assert torch.equal(g_dense(f, i), wd)
            assert g_sparse.replays == 8 and g_sparse.launches > 10
            # the replayed step inside the overlapped host-fed loop (its output buffers are reused)
            from ss_conv.pipeline import HostStream
            host = [(f.cpu().pin_memory(), i.cpu().pin_memory()) for f, i in batches]
            feed = HostStream(lambda f, i: (lambda y: (y.features, y.indices))(g_sparse(f, i)), cuda, cap,
                              step_reuses_outputs=True)
            got = [(of.clone(), oi.clone()) for of, oi in feed.run(iter(host * 2))]
            for (of, oi), (wf, wi, _) in zip(got, want * 2):
                assert torch.equal(oi, wi.cpu()) and torch.equal(of, wf.cpu())
            # two recordings: batches queued back to back, results read one batch late; the result of
            # a batch stays valid while the next one runs
            two = GraphedChain(sparse_net, [20] * 3, 3, 5, cap, cuda, depth=2, streams=2)
            queued, seen = [], []
            for f, i in batches * 2:
                queued.append(two.submit(f, i))
                if len(queued) >= 2:
                    y = queued[-2].result()
                    seen.append((y.features.clone(), y.indices.clone()))
            y = queued[-1].result()
            seen.append((y.features.clone(), y.indices.clone()))
            for (gf, gi), (wf, wi, _) in zip(seen, want * 2):
                assert torch.equal(gi, wi) and torch.equal(gf, wf)
            assert two.replays == 8 and two.fallbacks == 0
            # batches loaded once into the recordings' own input buffers and replayed in place
            two.load(0, *batches[2])
            two.load(1, *batches[0])
            for _ in range(2):
                qa, qb = two.submit_loaded(0), two.submit_loaded(1)
                ya, yb = qa.result(), qb.result()
                assert torch.equal(ya.indices, want[2][1]) and torch.equal(ya.features, want[2][0])
                assert torch.equal(yb.indices, want[0][1]) and torch.equal(yb.features, want[0][0])
            y = two(*batches[3])          # an ordinary call takes over recording 0 ...
            assert torch.equal(y.indices, want[3][1]) and torch.equal(y.features, want[3][0])
            yb = two.submit_loaded(1).result()   # ... and leaves the batch of recording 1 alone
            assert torch.equal(yb.indices, want[0][1]) and torch.equal(yb.features, want[0][0])
            # a much denser batch overflows the recorded capacities: exact fallback, then a new graph
            ind = S.bernoulli_voxels(range(3), 20, 0.45, base_seed=99)
            f, i = dev(S.features(ind.shape[0], 5, 7), cuda), dev(ind, cuda)
            big = GraphedChain(sparse_net, [20] * 3, 3, 5, ind.shape[0], cuda)
            big(*[t[:batches[1][1].shape[0]] for t in batches[1]])           # records with a sparse batch
            ref = sparse_net(SparseTensor(f, i, [20] * 3, 3))
            for _ in range(2):
                y = big(f, i)
                assert torch.equal(y.indices, ref.indices) and torch.equal(y.features, ref.features)
            # the same with two recordings and a queue: the overflowing batch is recomputed exactly,
            # the one queued behind it is not disturbed
            big2 = GraphedChain(sparse_net, [20] * 3, 3, 5, ind.shape[0], cuda, depth=2)
            small = [t[:batches[1][1].shape[0]] for t in batches[1]]
            big2(*small)
            qa, qb = big2.submit(f, i), big2.submit(*small)
            ya, yb = qa.result(), qb.result()
            assert torch.equal(ya.indices, ref.indices) and torch.equal(ya.features, ref.features)
            assert torch.equal(yb.indices, want[1][1]) and torch.equal(yb.features, want[1][0])
            assert big2.fallbacks <= 1        # 0 when the capacity hints raised by `big` above already cover the dense batch
        torch.cuda.synchronize()
        _ext.check_status(cuda)
    finally:
        _ext.set_precision("auto")


def test_voxelizer_count_stays_on_the_device_into_a_graphed_chain(cuda):
    """Point2Voxel hands out a tensor whose voxel count is still on the device; a GraphedChain
    takes it as it is (the count is checked after the replay).  Results equal the exact path."""
    from ss_conv import _ext
    from ss_conv.convolution import Convolution
    from ss_conv.graph import GraphedChain
    from ss_conv.pool import GlobalAvgPool
    from ss_conv.sp_ops.voxelize import Point2Voxel
    from ss_conv.utils import synthetic as S
    torch.manual_seed(6)
    p2v = Point2Voxel([16] * 3, [1.0 / 16] * 3, 4)
    conv = Convolution([(3, 0)], [(4, 0), (2, 1)], 3, stride=2, padding=1).to(cuda).eval()
    gpool = GlobalAvgPool()

    def net(x):
        return gpool(conv(x))

    _ext.set_precision("fp32")
    try:
        with torch.no_grad():
            g = None
            for r in range(3):
                pts, fts, ids = S.object_points(range(4), 600, base_seed=70 + 4 * r)
                P, Fe, I = dev(pts, cuda), dev(fts, cuda), dev(ids, cuda)
                x = p2v(P, Fe, I)[1]
                assert x.pending()
                if g is None:
                    g = GraphedChain(net, x.spatial_shape, x.batch_size, 3, 4 * 600, cuda)
                got = g(x).clone()
                old = _ext.AHEAD
                _ext.AHEAD = False
                try:
                    want = net(p2v(P, Fe, I)[1])
                finally:
                    _ext.AHEAD = old
                assert torch.equal(got, want)
            assert g.replays >= 2 and g.fallbacks == 0
        _ext.check_status(cuda)
    finally:
        _ext.set_precision("auto")


def test_ahead_path_edge_cases(cuda):
    """Capacity-sized layers on awkward inputs: a transposed convolution, an anisotropic kernel with
    dilation, a batch with an empty sample, a single voxel, and an empty tensor (which must take
    the exact path) - all bit-equal to the exact results."""
    from ss_conv import _ext
    from ss_conv.pool import AvgPool
    from ss_conv.sp_ops.conv import SparseConvolution
    from ss_conv.sp_ops.tensor import SparseTensor
    from ss_conv.utils import synthetic as S
    torch.manual_seed(8)
    layers = [SparseConvolution(3, 8, 12, 3, stride=2, padding=1, transposed=True, bias=False).to(cuda),
              SparseConvolution(3, 8, 12, (3, 1, 2), stride=1, padding=(2, 0, 1), dilation=(2, 1, 1), bias=True).to(cuda),
              AvgPool(3, stride=2, padding=1)]
    ind = S.bernoulli_voxels(range(3), 9, 0.2, base_seed=31)
    ind = ind[ind[:, 0] != 1]                                   # sample 1 is empty
    inputs = [(S.features(ind.shape[0], 8, 3), ind),
              (S.features(1, 8, 4), np.array([[2, 4, 4, 4]], dtype=np.int32)),
              (np.zeros((0, 8), np.float32), np.zeros((0, 4), np.int32))]
    _ext.set_precision("fp32")
    try:
        with torch.no_grad():
            for layer in layers:
                for feats, idx in inputs:
                    def run():
                        y = layer(SparseTensor(dev(feats, cuda), dev(idx, cuda), [9] * 3, 3))
                        return y.features.cpu().numpy(), y.indices.cpu().numpy()
                    old = _ext.AHEAD
                    _ext.AHEAD = False
                    try:
                        want = run()
                    finally:
                        _ext.AHEAD = old
                    run()                      # records the ratio (exact path)
                    got = run()                # capacity-sized path where it applies
                    np.testing.assert_array_equal(got[1], want[1])
                    np.testing.assert_array_equal(got[0], want[0])
        _ext.check_status(cuda)
    finally:
        _ext.set_precision("auto")


def test_plain24_backbone_replayed_as_one_graph(cuda):
    """The 24-block Plain24 backbone (three + twelve + nine SS_Conv blocks of 64 / 128 / 256 channels,
    three average pools) in eval mode: every module of submanifold blocks shares one rulebook, the row
    counts stay on the device from the first block to the last, so the whole network is recorded into
    ONE CUDA graph.  The replay gives the bits of the eager, exact-count pass, on the recorded batch and
    on another batch of different size."""
    from ss_conv import _ext
    from ss_conv.graph import GraphedChain
    from ss_conv.sp_ops.tensor import SparseTensor
    from ss_conv.utils import synthetic as S
    from ss_conv_backbones import Plain24
    torch.manual_seed(5)
    net = Plain24(irrep_in=(4,)).to(cuda).eval()
    V, B = 32, 4

    def batch(seed, n_pts):
        ind = S.surface_voxels(range(B), V, n_pts, base_seed=seed)
        g = torch.Generator(device="cpu").manual_seed(seed)
        return torch.randn(ind.shape[0], 4, generator=g).to(cuda), torch.from_numpy(ind).to(cuda)

    def last_stage(x):
        with torch.no_grad():
            return net(x)[3]

    def eager(f, i):
        old = _ext.AHEAD
        _ext.AHEAD = False
        try:
            y = last_stage(SparseTensor(f, i, [V] * 3, B))
            return y.features.clone(), y.indices.clone()
        finally:
            _ext.AHEAD = old

    _ext.set_precision("tf32")
    try:
        fa, ia = batch(100, 3000)
        fb, ib = batch(200, 2200)
        ref_a, ref_ia = eager(fa, ia)
        ref_b, ref_ib = eager(fb, ib)
        chain = GraphedChain(last_stage, [V] * 3, B, 4, int(max(ia.shape[0], ib.shape[0]) * 1.1), cuda)
        ya = chain(fa, ia)
        got_a, got_ia = ya.features.clone(), ya.indices.clone()
        yb = chain(fb, ib)
        got_b, got_ib = yb.features.clone(), yb.indices.clone()
    finally:
        _ext.set_precision("auto")
    _ext.check_status(cuda)
    assert chain.graph is not None and chain.launches >= 24 * 2 and chain.fallbacks == 0
    assert ya.spatial_shape[0] == V // 8 and got_a.shape[1] == 256
    assert torch.equal(got_ia, ref_ia) and torch.equal(got_ib, ref_ib)
    assert torch.equal(got_a, ref_a) and torch.equal(got_b, ref_b)
    assert float(ref_a.abs().max()) > 0


@pytest.mark.parametrize("storage", ["bf16", "fp16"])
def test_features_stored_in_16_bits_between_layers(cuda, storage):
    """set_feature_storage: a gated Activation writes fp16 / bf16 rows and the next convolution gathers
    them as its operands (no staging pass).  The stored rows are the rounding the staging pass would
    have produced, so a chain in storage mode gives the bits of the same chain with fp32 features and
    that operand precision - layer by layer, submanifold and strided, eager and as one CUDA graph."""
    from ss_conv import _ext
    from ss_conv.graph import GraphedChain
    from ss_conv.sp_ops.tensor import SparseTensor
    from ss_conv.utils import synthetic as S
    from ss_conv_modules import SS_Conv
    import torch.nn.functional as F
    torch.manual_seed(3)
    w = (4, 4, 4, 4)
    blocks = [SS_Conv(w, w, 3, padding=1, subm=True, activation=(F.relu, torch.sigmoid), indice_key="a",
                      activation_checkpoint=False).to(cuda).eval(),
              SS_Conv(w, w, 3, padding=1, subm=True, activation=(F.relu, torch.sigmoid), indice_key="a",
                      activation_checkpoint=False).to(cuda).eval(),
              SS_Conv(w, (8, 8, 8, 8), 3, stride=2, padding=1, activation=(F.relu, torch.sigmoid),
                      activation_checkpoint=False).to(cuda).eval()]
    ind = S.surface_voxels(range(3), 32, 5000, base_seed=77)
    feats = torch.randn(ind.shape[0], 64, generator=torch.Generator().manual_seed(1)).to(cuda)
    inds = torch.from_numpy(ind).to(cuda)

    def run(x):
        with torch.no_grad():
            for b in blocks:
                x = b(x)
        return x

    _ext.set_precision(storage)
    try:
        ref = run(SparseTensor(feats, inds, [32] * 3, 3))
        ref_f, ref_i = ref.features.clone(), ref.indices.clone()
        _ext.set_feature_storage(storage)
        l0 = _ext.kernel_launches()
        got = run(SparseTensor(feats, inds, [32] * 3, 3))
        got_f, got_i = got.features.clone(), got.indices.clone()
        l1 = _ext.kernel_launches()
        chain = GraphedChain(run, [32] * 3, 3, 64, int(ind.shape[0] * 1.1), cuda)
        rep = chain(feats, inds)
        rep_f = rep.features.clone()
    finally:
        _ext.set_feature_storage(None)
        _ext.set_precision("auto")
    _ext.check_status(cuda)
    dt = torch.bfloat16 if storage == "bf16" else torch.float16
    assert got_f.dtype == dt and got_f.shape == ref_f.shape and ref_f.dtype == torch.float32
    assert torch.equal(got_i, ref_i)
    assert torch.equal(got_f, ref_f.to(dt))          # same operands in every layer, only the last rounding differs
    assert torch.equal(rep_f, got_f)
    assert float(ref_f.abs().max()) > 0


def test_eval_batchnorm_refolds_when_its_buffers_change(cuda):
    """Eval-mode BatchNorm keeps the folded (scale, shift) of its running buffers between calls; an
    in-place change of a buffer or of the affine weight must be seen by the next call."""
    from ss_conv.batchnorm import BatchNorm
    from ss_conv.sp_ops.tensor import SparseTensor
    from ss_conv.utils import synthetic as S
    Rs = [(2, 0), (2, 1)]
    bn = BatchNorm(Rs).to(cuda).eval()
    ind = torch.from_numpy(S.surface_voxels(range(1), 16, 512, base_seed=2)).to(cuda)
    feats = torch.randn(ind.shape[0], 8, device=cuda)

    def run():
        with torch.no_grad():
            return bn(SparseTensor(feats.clone(), ind, [16] * 3, 1)).features.clone()

    a, again = run(), run()
    assert torch.equal(a, again)
    with torch.no_grad():
        bn.running_var.mul_(4.0)                 # in place: the fold must be redone
    b = run()
    assert not torch.equal(a, b) and torch.allclose(b, 0.5 * a, rtol=1e-4, atol=1e-5)
    with torch.no_grad():
        bn.weight.fill_(2.0)
    c = run()
    assert torch.allclose(c, 2.0 * b, rtol=1e-5, atol=1e-6)
