"""CPU restatement (numpy) of the SS-Conv sparse steerable convolution hot path.

TEST INFRASTRUCTURE ONLY: this module is the parity checker and the timed CPU baseline.
Nothing in the shipped package imports it; the product path is CUDA-only.

Every function cites the reference file:line (paths relative to the reference project
root) whose arithmetic it restates.  Parity pinning: the restatement is checked against
outputs of the reference's own C++/Python code (built by oracle/build_ref.py, fixtures
under tests/golden/ made by tests/golden/make_golden.py).  The steerable basis depends on
the third-party package `lie_learn` (unpinned, not vendored by the reference, not
installed): basis parity against a genuine lie_learn basis is UNPINNED; oracle and product
are always fed the same basis buffers, so layer parity does not depend on it.
"""
import numpy as np

I32 = np.int32


# ----------------------------------------------------------------------------- geometry
def conv_output_size(in_size, ksize, stride, padding, dilation):
    """SS_Conv_lib/ss_conv/sp_ops/ops.py:13-23."""
    out = []
    for n, k, s, p, d in zip(in_size, ksize, stride, padding, dilation):
        out.append(1 if k == -1 else (n + 2 * p - d * (k - 1) - 1) // s + 1)
    return out


def _as3(v):
    return [int(x) for x in v] if isinstance(v, (list, tuple, np.ndarray)) else [int(v)] * 3


def deconv_output_size(in_size, ksize, stride, padding, dilation, output_padding):
    """SS_Conv_lib/ss_conv/sp_ops/ops.py:26-36."""
    return [(n - 1) * s - 2 * p + k + op for n, k, s, p, op in zip(in_size, ksize, stride, padding, output_padding)]


def _candidate_pairs(indices, ksize, stride, padding, dilation, out_shape, transpose=False):
    """All (input row j, kernel offset kappa, output coord) triples allowed by
    SS_Conv_lib/src/conv/geometry.h:18-80 (getValidOutPos): out*stride - pad + k*dil == in,
    0 <= out < out_shape; kappa = (kx*ky_size + ky)*kz_size + kz (geometry.h:56-65).
    Returned sorted by (j, kappa), which is the reference CPU scan order
    (geometry.h:166-186: inputs ascending, candidates from the largest output coordinate
    downwards == ascending kappa).  For the transposed geometry the reference scans candidates
    from the largest output coordinate too, which is DEscending kappa; callers that need the
    reference's first-seen numbering there must not rely on this order (the rulebook parity
    tests compare in canonical order)."""
    n = indices.shape[0]
    kx, ky, kz = ksize
    K = kx * ky * kz
    js, ks, outs = [], [], []
    coords = indices[:, 1:4].astype(np.int64)
    for kappa in range(K):
        kk = (kappa // (ky * kz), (kappa // kz) % ky, kappa % kz)
        valid = np.ones(n, dtype=bool)
        o = np.empty((n, 3), dtype=np.int64)
        for d in range(3):
            if transpose:  # geometry.h:82-138 (getValidOutPosTranspose): out = in*stride - pad + k*dil
                od = coords[:, d] * stride[d] - padding[d] + kk[d] * dilation[d]
            else:
                num = coords[:, d] + padding[d] - kk[d] * dilation[d]
                valid &= (num % stride[d] == 0)
                od = num // stride[d]
            valid &= (od >= 0) & (od < out_shape[d])
            o[:, d] = od
        j = np.nonzero(valid)[0]
        js.append(j)
        ks.append(np.full(j.shape, kappa, dtype=np.int64))
        outs.append(o[j])
    j = np.concatenate(js) if js else np.zeros(0, np.int64)
    k = np.concatenate(ks) if ks else np.zeros(0, np.int64)
    o = np.concatenate(outs) if outs else np.zeros((0, 3), np.int64)
    order = np.lexsort((k, j))
    return j[order], k[order], o[order], K


def get_indice_pairs(indices, batch_size, spatial_shape, ksize=3, stride=1, padding=0, dilation=1,
                     subm=False, transpose=False, output_padding=0):
    """Rulebook in the reference's CPU order.

    Regular conv: SS_Conv_lib/src/conv/geometry.h:140-189 (getIndicePairsConv): outputs are
    numbered first-seen; pairs per offset in ascending input row; layout indicePairs[K,2,N]
    padded with -1, indiceNum[K] (SS_Conv_lib/src/conv/indice_conv.h:49-53).
    Submanifold: geometry.h:241-288 with the stride=1 / padding=k//2 override of
    indice_conv.h:68-73; output rows are the input rows (indice_conv.h:96).
    Returns (outids[Nout,4] int32, indicePairs[K,2,N] int32, indiceNum[K] int32).
    """
    indices = np.ascontiguousarray(indices, dtype=I32)
    ksize, stride, padding, dilation = _as3(ksize), _as3(stride), _as3(padding), _as3(dilation)
    spatial_shape = _as3(spatial_shape)
    n = indices.shape[0]
    if subm:
        stride = [1, 1, 1]
        padding = [k // 2 for k in ksize]
        out_shape = spatial_shape
    elif transpose:
        out_shape = deconv_output_size(spatial_shape, ksize, stride, padding, dilation, _as3(output_padding))
    else:
        out_shape = conv_output_size(spatial_shape, ksize, stride, padding, dilation)
    j, k, o, K = _candidate_pairs(indices, ksize, stride, padding, dilation, out_shape, transpose and not subm)
    assert K <= 256  # indice_conv.h:44
    vol = out_shape[0] * out_shape[1] * out_shape[2]
    b = indices[j, 0].astype(np.int64)
    flat = ((o[:, 0] * out_shape[1] + o[:, 1]) * out_shape[2] + o[:, 2]) + vol * b
    if subm:
        inflat = ((indices[:, 1].astype(np.int64) * out_shape[1] + indices[:, 2]) * out_shape[2]
                  + indices[:, 3]) + vol * indices[:, 0].astype(np.int64)
        order = np.argsort(inflat, kind="stable")
        sorted_flat = inflat[order]
        pos = np.searchsorted(sorted_flat, flat)
        pos_c = np.minimum(pos, max(n - 1, 0))
        hit = (sorted_flat[pos_c] == flat) if n else np.zeros(0, bool)
        # duplicates in the input: the reference's dense grid keeps the last writer (geometry.h:266-271)
        if n:
            last = np.searchsorted(sorted_flat, flat, side="right") - 1
            outrow = order[np.maximum(last, 0)]
        else:
            outrow = np.zeros(0, np.int64)
        j, k, outrow = j[hit], k[hit], outrow[hit]
        outids = indices
    else:
        uniq, first = np.unique(flat, return_index=True)
        rank_by_first = np.argsort(first, kind="stable")          # first-seen numbering
        number = np.empty(uniq.shape[0], dtype=np.int64)
        number[rank_by_first] = np.arange(uniq.shape[0])
        outrow = number[np.searchsorted(uniq, flat)]
        f = uniq[rank_by_first]
        outids = np.stack([f // vol, (f % vol) // (out_shape[1] * out_shape[2]),
                           (f // out_shape[2]) % out_shape[1], f % out_shape[2]], axis=1).astype(I32)
    pairs = np.full((K, 2, n), -1, dtype=I32)
    num = np.zeros(K, dtype=I32)
    order = np.lexsort((j, k))
    j, k, outrow = j[order], k[order], outrow[order]
    counts = np.bincount(k, minlength=K)
    start = 0
    for kappa in range(K):
        c = int(counts[kappa])
        pairs[kappa, 0, :c] = j[start:start + c]
        pairs[kappa, 1, :c] = outrow[start:start + c]
        num[kappa] = c
        start += c
    return outids, pairs, num


def canonical_rulebook(outids, pairs, num):
    """Order normalisation used by every rulebook parity test: renumber outputs by ascending
    (b,x,y,z) and sort each offset's pairs by input row.  The reference's CPU path numbers
    outputs first-seen (geometry.h:170-177), its GPU path by ascending flat index with
    atomic pair order (SS_Conv_lib/src/conv/indice_conv.h:120,
    SS_Conv_lib/src/conv/indice_cuda_functor.cu:23-66), so only this form is comparable."""
    outids = np.asarray(outids)
    pairs = np.asarray(pairs)
    num = np.asarray(num)
    order = np.lexsort((outids[:, 3], outids[:, 2], outids[:, 1], outids[:, 0]))
    new_of_old = np.empty(order.shape[0], dtype=np.int64)
    new_of_old[order] = np.arange(order.shape[0])
    can_out = outids[order]
    per_offset = []
    for kappa in range(pairs.shape[0]):
        c = int(num[kappa])
        i = pairs[kappa, 0, :c].astype(np.int64)
        o = new_of_old[pairs[kappa, 1, :c].astype(np.int64)]
        s = np.argsort(i, kind="stable")
        per_offset.append(np.stack([i[s], o[s]], axis=0).astype(I32))
    return can_out.astype(I32), per_offset, num.astype(I32)


def renumber_rows(outids):
    """Permutation `perm` with outids[perm] in ascending (b,x,y,z) order."""
    outids = np.asarray(outids)
    return np.lexsort((outids[:, 3], outids[:, 2], outids[:, 1], outids[:, 0]))


# --------------------------------------------------------------------- gather-GEMM-scatter
def indice_conv(features, filters, pairs, num, num_act_out, inverse=False, subm=False):
    """SS_Conv_lib/src/conv/indice_conv.h:247-343 (indiceConv<float>): for every kernel offset
    gather rows, multiply by filters[kappa] (Cin x Cout), scatter-add into the output; the
    submanifold centre (argmax of indiceNum, :259-262,283-286) is one dense product.
    `filters` is [K, Cin, Cout] (= the reference's [kx,ky,kz,Cin,Cout] viewed flat, :282)."""
    features = np.asarray(features, dtype=np.float32)
    filters = np.asarray(filters, dtype=np.float32).reshape(-1, features.shape[1], filters.shape[-1])
    K = pairs.shape[0]
    out = np.zeros((num_act_out, filters.shape[2]), dtype=np.float32)
    centre = int(np.argmax(num)) if K else 0
    if subm:
        out += features @ filters[centre]
    a, b = (1, 0) if inverse else (0, 1)
    for kappa in range(K):
        c = int(num[kappa])
        if c <= 0 or (subm and kappa == centre):
            continue
        buf = features[pairs[kappa, a, :c]] @ filters[kappa]
        np.add.at(out, pairs[kappa, b, :c], buf)
    return out


def indice_conv_f64(features, filters, pairs, num, num_act_out, inverse=False):
    """Same contraction in float64 (no submanifold shortcut): the error-free yardstick that
    tolerance tests normalise against."""
    features = np.asarray(features, dtype=np.float64)
    filters = np.asarray(filters, dtype=np.float64).reshape(-1, features.shape[1], filters.shape[-1])
    out = np.zeros((num_act_out, filters.shape[2]), dtype=np.float64)
    a, b = (1, 0) if inverse else (0, 1)
    for kappa in range(pairs.shape[0]):
        c = int(num[kappa])
        if c > 0:
            np.add.at(out, pairs[kappa, b, :c], features[pairs[kappa, a, :c]] @ filters[kappa])
    return out


def indice_conv_backward(features, filters, out_grad, pairs, num, inverse=False, subm=False, dtype=np.float32):
    """SS_Conv_lib/src/conv/indice_conv.h:344-426 (indiceConvBackward<float>): per kernel offset
    filtersGrad[kappa] = gathered(features)^T . gathered(outGrad) (:411) and the rows
    gathered(outGrad) . filters[kappa]^T are scatter-added into inputGrad (:412-424); the
    submanifold centre is two dense products (:373-377).  dtype=np.float64 gives the error-free
    yardstick for tolerance tests.  Returns (inputGrad [N,Cin], filtersGrad [K,Cin,Cout])."""
    features = np.asarray(features, dtype=dtype)
    out_grad = np.asarray(out_grad, dtype=dtype)
    flt = np.asarray(filters, dtype=dtype).reshape(-1, features.shape[1], np.shape(filters)[-1])
    K = pairs.shape[0]
    d_in = np.zeros_like(features)
    d_flt = np.zeros_like(flt)
    centre = int(np.argmax(num)) if K else 0
    if subm:
        d_flt[centre] = features.T @ out_grad
        d_in += out_grad @ flt[centre].T
    a, b = (1, 0) if inverse else (0, 1)
    for kappa in range(K):
        c = int(num[kappa])
        if c <= 0 or (subm and kappa == centre):
            continue
        fin = features[pairs[kappa, a, :c]]
        gout = out_grad[pairs[kappa, b, :c]]
        d_flt[kappa] = fin.T @ gout
        np.add.at(d_in, pairs[kappa, a, :c], gout @ flt[kappa].T)
    return d_in, d_flt


# ------------------------------------------------------------------------------- pooling
def indice_maxpool(features, pairs, num, num_act):
    """SS_Conv_lib/src/pool/indice_maxpool.h:15-50 + indice_maxpool_cpp_functor.cpp:16-40:
    output zero-initialised (:24), then out[o] = max(out[o], in[i]) per pair."""
    features = np.asarray(features, dtype=np.float32)
    out = np.zeros((num_act, features.shape[1]), dtype=np.float32)
    for kappa in range(pairs.shape[0]):
        c = int(num[kappa])
        if c > 0:
            np.maximum.at(out, pairs[kappa, 1, :c], features[pairs[kappa, 0, :c]])
    return out


def indice_maxpool_backward(features, out_features, out_grad, pairs, num):
    """SS_Conv_lib/src/pool/indice_maxpool_cpp_functor.cpp:65-86: for every pair and channel,
    din[i] += dout[o] where the input value equals the pooled value (ties all receive it)."""
    features = np.asarray(features, dtype=np.float32)
    d_in = np.zeros_like(features)
    for kappa in range(pairs.shape[0]):
        c = int(num[kappa])
        if c <= 0:
            continue
        i, o = pairs[kappa, 0, :c], pairs[kappa, 1, :c]
        np.add.at(d_in, i, np.where(out_features[o] == features[i], out_grad[o], np.float32(0)).astype(np.float32))
    return d_in


def indice_avgpool_backward(features, out_grad, pairs, num, summaryrf):
    """SS_Conv_lib/src/pool/indice_avgpool_cuda_functor.cu:175-205 (the reference has no CPU
    path, indice_avgpool.h:70-79): din[i] += dout[o] / rf[o] per pair, offsets ascending."""
    features = np.asarray(features, dtype=np.float32)
    d_in = np.zeros_like(features)
    rf = np.asarray(summaryrf).astype(np.float32)
    for kappa in range(pairs.shape[0]):
        c = int(num[kappa])
        if c <= 0:
            continue
        i, o = pairs[kappa, 0, :c], pairs[kappa, 1, :c]
        np.add.at(d_in, i, (out_grad[o] / rf[o][:, None]).astype(np.float32))
    return d_in


def global_avgpool_backward(d_out, offsets, n):
    """SS_Conv_lib/src/pool/global_avgpool_cuda_kernel.cu:45-59: every row of sample s receives
    d_out[s] / len(s)."""
    d_out = np.asarray(d_out, dtype=np.float32)
    d = np.zeros((n, d_out.shape[1]), dtype=np.float32)
    for s in range(len(offsets) - 1):
        lo, hi = int(offsets[s]), int(offsets[s + 1])
        if hi > lo:
            d[lo:hi] = d_out[s] / np.float32(hi - lo)
    return d


def global_maxpool_backward(d_out, maxidx, n):
    """SS_Conv_lib/src/pool/global_maxpool_cuda_kernel.cu:46-55: d_feats[argmax row, c] += d_out[s, c]."""
    d_out = np.asarray(d_out, dtype=np.float32)
    d = np.zeros((n, d_out.shape[1]), dtype=np.float32)
    for s in range(d_out.shape[0]):
        for c in range(d_out.shape[1]):
            if maxidx[s, c] >= 0:
                d[maxidx[s, c], c] += d_out[s, c]
    return d


def summary_rf(pairs, num, num_act):
    """SS_Conv_lib/src/pool/indiceSummaryRF.cu:21-36: number of present inputs per output."""
    rf = np.zeros(num_act, dtype=I32)
    for kappa in range(pairs.shape[0]):
        c = int(num[kappa])
        if c > 0:
            np.add.at(rf, pairs[kappa, 1, :c], 1)
    return rf


def indice_avgpool(features, pairs, num, num_act, summaryrf=None):
    """SS_Conv_lib/src/pool/indice_avgpool_cuda_functor.cu:21-53: out[o] += in[i] / rf[o],
    offsets processed in ascending order (indice_avgpool.h:28-47).  With the Python default
    use_gs=True the divisor is the kernel volume for every row
    (SS_Conv_lib/ss_conv/sp_ops/functional.py:171-176)."""
    features = np.asarray(features, dtype=np.float32)
    if summaryrf is None:
        summaryrf = np.full(num_act, pairs.shape[0], dtype=I32)
    out = np.zeros((num_act, features.shape[1]), dtype=np.float32)
    for kappa in range(pairs.shape[0]):
        c = int(num[kappa])
        if c > 0:
            o = pairs[kappa, 1, :c]
            term = features[pairs[kappa, 0, :c]] / summaryrf[o].astype(np.float32)[:, None]
            out[o] = out[o] + term        # each output row occurs at most once per offset
    return out


def global_avgpool(feats, offsets):
    """SS_Conv_lib/src/pool/global_avgpool_cuda_kernel.cu:16-34: sequential fp32 row sum per
    (sample, channel) divided by the row count (empty sample -> 0/0 = NaN)."""
    feats = np.asarray(feats, dtype=np.float32)
    B = len(offsets) - 1
    out = np.zeros((B, feats.shape[1]), dtype=np.float32)
    for s in range(B):
        a, b = int(offsets[s]), int(offsets[s + 1])
        acc = np.zeros(feats.shape[1], dtype=np.float32)
        for r in range(a, b):
            acc = acc + feats[r]
        with np.errstate(invalid="ignore", divide="ignore"):
            out[s] = acc / np.float32(b - a)
    return out


def global_maxpool(feats, offsets):
    """SS_Conv_lib/src/pool/global_maxpool_cuda_kernel.cu:16-35: per (sample, channel) max and
    first arg-max row (strict >, initial value -inf, arg -1)."""
    feats = np.asarray(feats, dtype=np.float32)
    B = len(offsets) - 1
    out = np.full((B, feats.shape[1]), -np.inf, dtype=np.float32)
    arg = np.full((B, feats.shape[1]), -1, dtype=I32)
    for s in range(B):
        a, b = int(offsets[s]), int(offsets[s + 1])
        if b > a:
            seg = feats[a:b]
            out[s] = seg.max(axis=0)
            arg[s] = a + seg.argmax(axis=0)
    return out, arg


# --------------------------------------------------------------------------- voxelization
def voxel2point_map(inverse, n_active, max_active, mode):
    """SS_Conv_lib/src/voxelize/voxel2point_cuda_kernel.cu:16-37 with the initial values of
    SS_Conv_lib/ss_conv/sp_ops/functional.py:344-351.  Row v = [count, point ids...].
    Modes 3/4 append ids in atomic order in the reference; here ascending point id (the
    deterministic representative; compare rows as sets)."""
    inverse = np.asarray(inverse).reshape(-1)
    n = inverse.shape[0]
    if mode in (3, 4):
        maps = np.zeros((n_active, max_active + 1), dtype=I32)
        for pid in range(n):
            v = inverse[pid]
            c = maps[v, 0]
            maps[v, c + 1] = pid
            maps[v, 0] = c + 1
    elif mode == 2:
        maps = np.full((n_active, max_active + 1), -1, dtype=I32)
        np.maximum.at(maps[:, 1], inverse, np.arange(n, dtype=I32))
        maps[inverse, 0] = 1
    elif mode == 1:
        maps = np.full((n_active, max_active + 1), n, dtype=I32)
        np.minimum.at(maps[:, 1], inverse, np.arange(n, dtype=I32))
        maps[inverse, 0] = 1
    else:
        raise ValueError("mode must be 1..4")
    return maps


def voxelize_fp(feats, maps, mode):
    """SS_Conv_lib/src/voxelize/voxelize_cuda_kernel.h:18-32: out[v] = sum_i mult*feats[map[v,i]],
    mult = 1/count only for mode 4 (SS_Conv_lib/src/voxelize/voxelize.h:90)."""
    feats = np.asarray(feats, dtype=np.float32)
    M = maps.shape[0]
    out = np.zeros((M, feats.shape[1]), dtype=np.float32)
    for v in range(M):
        c = int(maps[v, 0])
        mult = np.float32(1) / np.float32(c) if (mode == 4 and c > 0) else np.float32(1)
        for i in range(1, c + 1):
            out[v] = out[v] + mult * feats[maps[v, i]]
    return out


def point2voxel(points, feats, batch_ids, voxel_num_limit, unit_voxel_extent, mode=4):
    """SS_Conv_lib/ss_conv/sp_ops/voxelize.py:29-99 restricted to the case where every sample
    keeps at least one in-range point (the empty-sample branch :63-78 injects a zero point).
    Returns (valid_points, voxel_feats, voxel_indices[M,4], valid_ids, inverse)."""
    points = np.asarray(points, dtype=np.float32)
    feats = np.asarray(feats, dtype=np.float32)
    unit = np.asarray(unit_voxel_extent, dtype=np.float32).reshape(1, 3)
    lim = np.asarray(voxel_num_limit, dtype=np.float32).reshape(1, 3)
    half = np.float32(0.5) * (lim * unit)
    keep = (np.abs(points) > half).sum(1) == 0
    p, f, ids = points[keep], feats[keep], np.asarray(batch_ids)[keep]
    order = np.argsort(ids, kind="stable")
    p, f, ids = p[order], f[order], ids[order]
    vi = ((p + half) / unit).astype(I32)
    key = np.concatenate([ids.reshape(-1, 1).astype(I32), vi], axis=1)
    occupied, inverse, count = np.unique(key, axis=0, return_inverse=True, return_counts=True)
    inverse = inverse.reshape(-1)
    max_active = 1 if mode in (1, 2) else int(count.max())
    maps = voxel2point_map(inverse, occupied.shape[0], max_active, mode)
    return p, voxelize_fp(f, maps, mode), occupied.astype(I32), ids, inverse.astype(I32)


def _fma32(a, b, c):
    """fp32 fused multiply-add a*b + c: the product of two fp32 values is exact in float64, the
    sum is rounded to float64 and then to fp32 (double rounding can differ from a true fma only
    when the float64 sum lands exactly on an fp32 rounding boundary)."""
    return (np.asarray(a, np.float32).astype(np.float64) * np.asarray(b, np.float32).astype(np.float64)
            + np.asarray(c, np.float32).astype(np.float64)).astype(np.float32)


def three_nn(unknown, known):
    """SS_Conv_lib/src/voxelize/interpolate_cuda_kernel.cu:8-55: per query (b,x,y,z) scan all
    known rows of the same batch id, fp32 squared distance, keep the three smallest with
    strict < (first index wins ties); unfilled slots keep 1e40 (-> +inf in fp32) and index 0.
    The distance dx*dx + dy*dy + dz*dz (:39) is evaluated as nvcc contracts it,
    fma(dz, dz, fma(dx, dx, dy*dy)): pinned bit for bit to the reference's compiled kernel."""
    unknown = np.asarray(unknown, dtype=np.float32)
    known = np.asarray(known, dtype=np.float32)
    n = unknown.shape[0]
    dist2 = np.empty((n, 3), dtype=np.float32)
    idx = np.zeros((n, 3), dtype=I32)
    for q in range(n):
        same = np.nonzero(known[:, 0] == unknown[q, 0])[0]
        dx = unknown[q, 1] - known[same, 1]
        dy = unknown[q, 2] - known[same, 2]
        dz = unknown[q, 3] - known[same, 3]
        d = _fma32(dz, dz, _fma32(dx, dx, dy * dy))
        order = np.argsort(d, kind="stable")[:3]
        best = np.full(3, np.inf, dtype=np.float32)
        bi = np.zeros(3, dtype=I32)
        best[:order.shape[0]] = d[order]
        bi[:order.shape[0]] = same[order]
        dist2[q], idx[q] = best, bi
    return dist2, idx


def three_interpolate(points, idx, weight):
    """SS_Conv_lib/src/voxelize/interpolate_cuda_kernel.cu:79-101:
    out[n,c] = w0*p[i0,c] + w1*p[i1,c] + w2*p[i2,c], evaluated as nvcc contracts it,
    fma(w2, p2, fma(w0, p0, w1*p1)): pinned bit for bit to the reference's compiled kernel."""
    points = np.asarray(points, dtype=np.float32)
    weight = np.asarray(weight, dtype=np.float32)
    t = _fma32(weight[:, 0:1], points[idx[:, 0]], weight[:, 1:2] * points[idx[:, 1]])
    return _fma32(weight[:, 2:3], points[idx[:, 2]], t)


def voxel2point(voxel_feats, voxel_indices, spatial_shape, unit_voxel_extent, points, batch_ids):
    """SS_Conv_lib/ss_conv/sp_ops/voxelize.py:127-162: voxel centres idx*unit - extent/2 + unit/2,
    3-NN, weights 1/(sqrt(d2)+1e-8) normalised, interpolation."""
    unit = np.asarray(unit_voxel_extent, dtype=np.float32)
    extent = (np.asarray(unit_voxel_extent, dtype=np.float64) * np.asarray(spatial_shape, dtype=np.float64)).astype(np.float32)
    known = np.asarray(voxel_indices).astype(np.float32)
    known[:, 1:] = known[:, 1:] * unit - np.float32(0.5) * extent + np.float32(0.5) * unit
    unknown = np.concatenate([np.asarray(batch_ids, dtype=np.float32).reshape(-1, 1),
                              np.asarray(points, dtype=np.float32)], axis=1)
    d2, idx = three_nn(unknown, known)
    recip = np.float32(1.0) / (np.sqrt(d2) + np.float32(1e-8))
    w = recip / recip.sum(1, keepdims=True)
    return three_interpolate(voxel_feats, idx, w), d2, idx


# --------------------------------------------------------------- irrep-wise BN / activation
def rs_dim(Rs):
    """SS_Conv_lib/ss_conv/utils/utils.py:6-10."""
    return sum(m * (2 * l + 1) for m, l in Rs)


def batchnorm_eval(x, Rs, running_mean, running_var, weight, bias, eps=1e-5):
    """SS_Conv_lib/ss_conv/batchnorm.py:49-115 in eval mode (running statistics)."""
    x = np.asarray(x, dtype=np.float32)
    out = np.empty_like(x)
    ix = irm = irv = 0
    for m, l in Rs:
        d = 2 * l + 1
        f = x[:, ix:ix + m * d].reshape(-1, m, d)
        if d == 1:
            f = f - running_mean[irm:irm + m].reshape(1, m, 1)
        scale = np.power(running_var[irv:irv + m] + np.float32(eps), np.float32(-0.5)).astype(np.float32)
        if weight is not None:
            scale = scale * weight[irv:irv + m]
        f = f * scale.reshape(1, m, 1)
        if d == 1 and bias is not None:
            f = f + bias[irm:irm + m].reshape(1, m, 1)
        out[:, ix:ix + m * d] = f.reshape(-1, m * d)
        if d == 1:
            irm += m
        irv += m
        ix += m * d
    return out


def batchnorm_train(x, Rs, running_mean, running_var, weight, bias, eps=1e-5, momentum=0.1):
    """SS_Conv_lib/ss_conv/batchnorm.py:49-136 in training mode: scalars use batch mean and
    mean of squared deviations, non-scalars the batch mean of the squared field norm;
    running statistics move by `momentum` (:45-46).  Returns (y, new_mean, new_var)."""
    x = np.asarray(x, dtype=np.float32)
    out = np.empty_like(x)
    new_mean, new_var = running_mean.copy(), running_var.copy()
    ix = irm = irv = 0
    for m, l in Rs:
        d = 2 * l + 1
        f = x[:, ix:ix + m * d].reshape(-1, m, d)
        if d == 1:
            mu = f.mean(0).reshape(-1)
            new_mean[irm:irm + m] = (1 - momentum) * running_mean[irm:irm + m] + momentum * mu
            f = f - mu.reshape(1, m, 1)
        norm = (f ** 2).sum(2).mean(0)
        new_var[irv:irv + m] = (1 - momentum) * running_var[irv:irv + m] + momentum * norm
        scale = np.power(norm + np.float32(eps), np.float32(-0.5)).astype(np.float32)
        if weight is not None:
            scale = scale * weight[irv:irv + m]
        f = f * scale.reshape(1, m, 1)
        if d == 1 and bias is not None:
            f = f + bias[irm:irm + m].reshape(1, m, 1)
        out[:, ix:ix + m * d] = f.reshape(-1, m * d)
        if d == 1:
            irm += m
        irv += m
        ix += m * d
    return out, new_mean, new_var


def _act(name, v):
    if name == "relu":
        return np.maximum(v, np.float32(0))
    if name == "sigmoid":
        return (np.float32(1) / (np.float32(1) + np.exp(-v))).astype(np.float32)
    if name in (None, "identity"):
        return v
    raise ValueError(name)


def gated_activation(y, Rs, scalar_act="relu", gate_act="sigmoid", scalar_bias=None, gate_bias=None):
    """SS_Conv_lib/ss_conv/activation.py:55-100,130-160: input [N, C+G] -> output [N, C]; the
    first Rs entry (l==0) goes through the scalar activation, every l>0 field is multiplied
    by its activated gate scalar taken from the trailing G channels in Rs order."""
    y = np.asarray(y, dtype=np.float32)
    C = rs_dim(Rs)
    out = np.empty((y.shape[0], C), dtype=np.float32)
    mult = [m for m, _ in Rs]
    use_scalar = scalar_act is not None and mult[0] > 0 and Rs[0][1] == 0
    n_gate = sum(mult[1:])
    use_gate = gate_act is not None and n_gate > 0
    if use_gate:
        g = y[:, C:C + n_gate]
        if gate_bias is not None:
            g = g + gate_bias.reshape(1, -1)
        g = _act(gate_act, g)
    by = bg = 0
    for m, l in Rs:
        if m == 0:
            continue
        d = 2 * l + 1
        f = y[:, by:by + m * d]
        if l == 0:
            if use_scalar:
                if scalar_bias is not None:
                    f = f + scalar_bias.reshape(1, -1)
                f = _act(scalar_act, f)
        elif use_gate:
            f = (f.reshape(-1, m, d) * g[:, bg:bg + m].reshape(-1, m, 1)).reshape(-1, m * d)
            bg += m
        out[:, by:by + m * d] = f
        by += m * d
    return out


# ------------------------------------------------------------------ kernel materialisation
def combination(weight, bases, Rs_in, Rs_out, size):
    """SS_Conv_lib/ss_conv/utils/kernel.py:267-299: W[c_out(i,u)+a, c_in(j,v)+c, x,y,z] =
    sum_b w_ij[u,v,b] * B_ij[b,a,c,x,y,z]; weight segments consumed i-outer / j-inner;
    a missing basis gives a zero block (:286-290).  `bases[(i,j)]` is an array or None.
    Returns [Cout, Cin, k, k, k] float32."""
    rows = []
    wi = 0
    for i, (mo, lo) in enumerate(Rs_out):
        cols = []
        for j, (mi, li) in enumerate(Rs_in):
            B = bases[(i, j)]
            if B is not None:
                nb = B.shape[0]
                w = np.asarray(weight[wi:wi + mo * mi * nb], dtype=np.float32).reshape(mo, mi, nb)
                wi += mo * mi * nb
                ker = np.einsum("uvb,bijxyz->uivjxyz", w, B.astype(np.float32)).astype(np.float32)
                ker = ker.reshape(mo * (2 * lo + 1), mi * (2 * li + 1), size, size, size)
            else:
                ker = np.zeros((mo * (2 * lo + 1), mi * (2 * li + 1), size, size, size), np.float32)
            cols.append(ker)
        rows.append(np.concatenate(cols, axis=1))
    assert wi == len(weight)
    return np.concatenate(rows, axis=0)


def filters_from_kernel(W):
    """SS_Conv_lib/ss_conv/convolution.py:56: [Cout,Cin,kx,ky,kz] -> [kx,ky,kz,Cin,Cout]."""
    return np.ascontiguousarray(np.transpose(W, (2, 3, 4, 1, 0)))


# ----------------------------------------------------------------- voxelizer gradients
def voxelize_bp(d_out, maps, mode, n_point):
    """SS_Conv_lib/src/voxelize/voxelize_cuda_kernel.h:44-57: every point listed in a voxel's
    rule row [count, ids...] receives the voxel's gradient, times 1/count in mean mode 4."""
    d_out = np.asarray(d_out, dtype=np.float32)
    d = np.zeros((n_point, d_out.shape[1]), dtype=np.float32)
    for v in range(maps.shape[0]):
        n_act = int(maps[v, 0])
        mult = np.float32(1.0 / n_act) if (mode == 4 and n_act > 0) else np.float32(1.0)
        for p in maps[v, 1:1 + n_act]:
            d[p] += mult * d_out[v]
    return d


def three_interpolate_bp(grad_out, idx, weight, m):
    """SS_Conv_lib/src/voxelize/interpolate_cuda_kernel.cu:123-145:
    grad_points[idx[p, j]] += grad_out[p] * weight[p, j] (float64 accumulation here)."""
    g = np.zeros((m, grad_out.shape[1]), dtype=np.float64)
    for j in range(3):
        np.add.at(g, idx[:, j], grad_out.astype(np.float64) * weight[:, j:j + 1].astype(np.float64))
    return g


# ------------------------------------------------------------------------ feature steering
def steer_points(points, ids, rot, trans, scale=None):
    """Common_utils/ss_conv_modules.py:198-208 (_transform_points): (p - t_b) @ R_b, divided by
    (s_b + 1e-8) when a scale is given."""
    p = (np.asarray(points, np.float32) - trans[ids])[:, None, :] @ rot[ids]
    p = p[:, 0, :]
    if scale is not None:
        p = p / (np.asarray(scale, np.float32)[ids].reshape(-1, 1) + np.float32(1e-8))
    return p.astype(np.float32)


def steer_feats(feats, ids, d_mats, irrep):
    """Common_utils/ss_conv_modules.py:210-224 (_transform_feats): every copy of every order-l
    block of a feature row is multiplied from the right by D^l of the row's sample
    (d_mats[l]: [B, 2l+1, 2l+1])."""
    f = np.asarray(feats, np.float32)
    out = np.empty_like(f)
    dim = 0
    for l, m in enumerate(irrep):
        D = np.asarray(d_mats[l], np.float32)[ids]
        for _ in range(int(m)):
            w = 2 * l + 1
            out[:, dim:dim + w] = (f[:, None, dim:dim + w] @ D)[:, 0, :]
            dim += w
    assert dim == f.shape[1]
    return out
